// Kernels for what a sequence carries from token to token besides keys and values: the
// previous token of a hashed bigram embedding, the previous rows of a token shift or a short
// convolution; and the small row-wise steps of decoders that need them: the input of a pass
// over a looped stretch of layers, GELU, the soft cap of logits, the mean of several normed
// branch outputs.
//
// A step's rows are packed: sequence s owns rows seq_row0[s] .. + seq_new[s]; row r belongs to
// row_seq[r] and stands at position row_pos[r]; the state of sequence s lies at seq_slot[s].
// A kernel that reads state and one that replaces it are separate launches, so a step of many
// rows never reads what it has just written. All arithmetic in float.
#include "common.cuh"

// ------------------------------------------------------------------------------------
// out[r] = table[tok] + bigram[(prev * mul_prev + tok * mul_cur) mod buckets]; the row
// `buckets` for a sequence's first token. prev is the token of the row before, or, for the
// first row of a step, what `prev_state[slot]` kept. bigram may be null (plain embedding).
template <typename T>
__global__ void bigram_embed_kernel(const T* __restrict__ table, const T* __restrict__ bigram, const int* __restrict__ tokens,
                                    const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                    const int* __restrict__ seq_row0, const int* __restrict__ seq_slot,
                                    const int* __restrict__ prev_state, float* __restrict__ out, int hidden, int vocab,
                                    long long buckets, long long mul_prev, long long mul_cur, int* err) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tok = tokens[r];
    float* o = out + (size_t)r * hidden;
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, 1);
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = 0.f;
        return;
    }
    const T* src = table + (size_t)tok * hidden;
    if (!bigram) {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = to_f32(src[c]);
        return;
    }
    const int s = row_seq[r];
    long long brow = buckets;
    if (row_pos[r] > 0) {
        const int prev = r > seq_row0[s] ? tokens[r - 1] : prev_state[seq_slot[s]];
        brow = ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
        if (brow < 0) brow += buckets;
    }
    const T* b = bigram + (size_t)brow * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = to_f32(src[c]) + to_f32(b[c]);
}

// prev_state[slot of s] = the last token sequence s brought in this step.
__global__ void keep_last_token_kernel(const int* __restrict__ tokens, const int* __restrict__ seq_row0,
                                       const int* __restrict__ seq_new, const int* __restrict__ seq_slot,
                                       int* __restrict__ prev_state, int n_seqs) {
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < n_seqs) prev_state[seq_slot[s]] = tokens[seq_row0[s] + seq_new[s] - 1];
}

extern "C" int cml_bigram_embed(const void* table, const void* bigram, int dtype, const int* tokens, const int* row_seq,
                                const int* row_pos, const int* seq_row0, const int* seq_new, const int* seq_slot,
                                int* prev_state, float* out, int rows, int n_seqs, int hidden, int vocab, long long buckets,
                                long long mul_prev, long long mul_cur, int* err, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = hidden >= 1024 ? 256 : 128;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(bigram_embed_kernel<float>, dim3(rows), dim3(block), 0, s, (const float*)table, (const float*)bigram, tokens,
                   row_seq, row_pos, seq_row0, seq_slot, (const int*)prev_state, out, hidden, vocab, buckets, mul_prev, mul_cur, err);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(bigram_embed_kernel<bf16>, dim3(rows), dim3(block), 0, s, (const bf16*)table, (const bf16*)bigram, tokens,
                   row_seq, row_pos, seq_row0, seq_slot, (const int*)prev_state, out, hidden, vocab, buckets, mul_prev, mul_cur, err);
    else
        return CML_ERR_BAD_DTYPE;
    if (bigram)
        launch_pdl(keep_last_token_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, s, tokens, seq_row0, seq_new, seq_slot,
                   prev_state, n_seqs);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// state[slot, j, c] (j < keep) = the value of column col0 + c of the sequence's (keep - j)-th
// last row after this step: a row of this step where it brought that many, else what the state
// held (zeros for a sequence that starts here). A thread owns one column of one sequence.
template <typename T>
__global__ void keep_last_rows_kernel(const T* __restrict__ src, long ld, int col0, int width, int keep,
                                      const int* __restrict__ seq_row0, const int* __restrict__ seq_new,
                                      const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                                      float* __restrict__ state) {
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int n = seq_new[s], row0 = seq_row0[s];
    const bool fresh = seq_start[s] == 0;
    float* st = state + (size_t)seq_slot[s] * keep * width + c;
    for (int j = 0; j < keep; ++j) {
        const int o = n - keep + j;                       // offset of that row among the step's rows
        float v;
        if (o >= 0) v = to_f32(src[(size_t)(row0 + o) * ld + col0 + c]);
        else v = fresh ? 0.f : st[(size_t)(n + j) * width];
        st[(size_t)j * width] = v;
    }
}

extern "C" int cml_keep_last_rows(const void* src, int dtype, long ld, int col0, int width, int keep, const int* seq_row0,
                                  const int* seq_new, const int* seq_start, const int* seq_slot, float* state, int n_seqs,
                                  void* stream) {
    if (n_seqs <= 0 || width <= 0 || keep <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((width + 127) / 128, n_seqs);
    if (dtype == CML_DTYPE_F32)
        launch_pdl(keep_last_rows_kernel<float>, grid, dim3(128), 0, s, (const float*)src, ld, col0, width, keep, seq_row0, seq_new,
                   seq_start, seq_slot, state);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(keep_last_rows_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)src, ld, col0, width, keep, seq_row0, seq_new,
                   seq_start, seq_slot, state);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// Token shift: out[r] = h[r] + (h'[r] - h[r]) * mix, h' the row before of the same sequence
// (zeros for the first token; state[slot] for the first row of a later step).
template <typename T, typename TW>
__global__ void token_shift_kernel(const T* __restrict__ h, const TW* __restrict__ mix, const float* __restrict__ state,
                                   const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                   const int* __restrict__ seq_row0, const int* __restrict__ seq_slot, T* __restrict__ out,
                                   int hidden) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int s = row_seq[r];
    const bool first = row_pos[r] == 0, inside = r > seq_row0[s];
    const T* cur = h + (size_t)r * hidden;
    const T* before = h + (size_t)(inside ? r - 1 : r) * hidden;
    const float* st = state + (size_t)seq_slot[s] * hidden;
    T* o = out + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float x = to_f32(cur[c]);
        const float p = first ? 0.f : (inside ? to_f32(before[c]) : st[c]);
        o[c] = from_f32<T>(x + (p - x) * to_f32(mix[c]));
    }
}

extern "C" int cml_token_shift(const void* h, int dtype, const void* mix, int mix_dtype, const float* state, const int* row_seq,
                               const int* row_pos, const int* seq_row0, const int* seq_slot, void* out, int rows, int hidden,
                               void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = hidden >= 1024 ? 256 : 128;
#define TS_CASE(T_, TW_, D_, DW_)                                                                                         \
    if (dtype == D_ && mix_dtype == DW_) {                                                                                \
        launch_pdl(token_shift_kernel<T_, TW_>, dim3(rows), dim3(block), 0, s, (const T_*)h, (const TW_*)mix, state, row_seq, \
                   row_pos, seq_row0, seq_slot, (T_*)out, hidden);                                                         \
        return cml_launch_status();                                                                                       \
    }
    TS_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    TS_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    TS_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    TS_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
#undef TS_CASE
    return CML_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------
// One-token steps: RMS norm and token shift in one launch. Row r is the one new row of sequence
// row_seq[r], so one block reads the sequence's kept row and replaces it. x[r] += the pending
// split sums (in split order, written back); n = x[r] / sqrt(mean + eps) * w rounded to the
// compute type; out[r] = n + (kept - n) * mix (kept: zeros at position 0); kept <- n.
// The arithmetic is that of the three separate kernels.
template <typename TW, typename T>
__global__ void rmsnorm_shift_kernel(float* __restrict__ x, const TW* __restrict__ w, const float* __restrict__ mix,
                                     float* __restrict__ state, const int* __restrict__ row_seq,
                                     const int* __restrict__ row_pos, const int* __restrict__ seq_slot, T* __restrict__ out,
                                     int hidden, float eps, const float* __restrict__ partial, int n_splits,
                                     size_t split_stride) {
    __shared__ float red[33];
    extern __shared__ float rowbuf[];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * hidden;
    float ss = 0.f;
    // two columns of a thread at a time; the row's values and sixteen splits of both are in flight together
    // (every load unconditional, of a valid place), the adds in split order
    for (int cb = threadIdx.x; cb < hidden; cb += 2 * blockDim.x) {
        const int cc[2] = {cb, cb + (int)blockDim.x};
        const bool in[2] = {true, cc[1] < hidden};
        float v[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) v[j] = xr[in[j] ? cc[j] : cb];
        if (partial) {
            for (int s0 = 0; s0 < n_splits; s0 += 16) {
                float t[2][16];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float* pp = partial + (size_t)r * hidden + (in[j] ? cc[j] : cb);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float tv = pp[(size_t)min(s0 + i, n_splits - 1) * split_stride];
                        t[j][i] = s0 + i < n_splits ? tv : 0.f;
                    }
                }
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[j] += t[j][i];
            }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (!in[j]) continue;
            if (partial) xr[cc[j]] = v[j];
            rowbuf[cc[j]] = v[j];
            ss = fmaf(v[j], v[j], ss);
        }
    }
    const bool first = row_pos[r] == 0;
    float* st = state + (size_t)seq_slot[row_seq[r]] * hidden;
    // what the second pass needs besides the row's scale is asked for before the reduction
    const int c0 = threadIdx.x, c1 = threadIdx.x + blockDim.x;
    const int a0 = c0 < hidden ? c0 : 0, a1 = c1 < hidden ? c1 : 0;
    const float w0 = to_f32(w[a0]), w1 = to_f32(w[a1]), m0 = mix[a0], m1 = mix[a1], k0 = st[a0], k1 = st[a1];
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* o = out + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float wc = c == c0 ? w0 : (c == c1 ? w1 : to_f32(w[c]));
        const float mc = c == c0 ? m0 : (c == c1 ? m1 : mix[c]);
        const float kc = c == c0 ? k0 : (c == c1 ? k1 : st[c]);
        const float n = to_f32(from_f32<T>(rowbuf[c] * scale * wc));
        const float kept = first ? 0.f : kc;
        o[c] = from_f32<T>(n + (kept - n) * mc);
        st[c] = n;
    }
}

extern "C" int cml_rmsnorm_shift(float* x, const void* w, int w_dtype, const float* mix, float* state, const int* row_seq,
                                 const int* row_pos, const int* seq_slot, void* out, int out_dtype, int rows, int hidden,
                                 float eps, const float* partial, int n_splits, long split_stride, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = hidden >= 2048 ? 1024 : (hidden >= 512 ? 256 : 128);
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024) return CML_ERR_BAD_SIZE;
#define RS_CASE(TW_, T_, DW_, D_)                                                                                           \
    if (w_dtype == DW_ && out_dtype == D_) {                                                                                \
        launch_pdl(rmsnorm_shift_kernel<TW_, T_>, dim3(rows), dim3(block), smem, s, x, (const TW_*)w, mix, state, row_seq, row_pos, \
                   seq_slot, (T_*)out, hidden, eps, partial, n_splits, (size_t)split_stride);                              \
        return cml_launch_status();                                                                                         \
    }
    RS_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    RS_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
    RS_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    RS_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
#undef RS_CASE
    return CML_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------
// h[r] += (base ? base[r] : 0) + vec: the input of one pass over a looped stretch.
template <typename TW>
__global__ void add_rows_vec_kernel(float* __restrict__ h, const float* __restrict__ base, const TW* __restrict__ vec,
                                    long n, int hidden) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        float v = h[i];
        if (base) v += base[i];
        h[i] = v + to_f32(vec[i % hidden]);
    }
}

extern "C" int cml_add_rows_vec(float* h, const float* base, const void* vec, int vec_dtype, int rows, int hidden, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long n = (long)rows * hidden;
    const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (vec_dtype == CML_DTYPE_F32)
        launch_pdl(add_rows_vec_kernel<float>, dim3(grid), dim3(256), 0, s, h, base, (const float*)vec, n, hidden);
    else if (vec_dtype == CML_DTYPE_BF16)
        launch_pdl(add_rows_vec_kernel<bf16>, dim3(grid), dim3(256), 0, s, h, base, (const bf16*)vec, n, hidden);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// x = 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))) in place.
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
template <typename T>
__global__ void gelu_tanh_kernel(T* __restrict__ x, long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        x[i] = from_f32<T>(gelu_tanh_f(to_f32(x[i])));
}

extern "C" int cml_gelu_tanh(void* x, int dtype, long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    if (dtype == CML_DTYPE_F32) launch_pdl(gelu_tanh_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)x, n);
    else if (dtype == CML_DTYPE_BF16) launch_pdl(gelu_tanh_kernel<bf16>, dim3(grid), dim3(256), 0, s, (bf16*)x, n);
    else return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// The activations of the dense feed-forwards: 0 none, 1 GELU (tanh form), 2 the square of ReLU, 3 GELU (exact,
// 0.5 z (1 + erf(z / sqrt 2))).
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return gelu_tanh_f(v);
    if (act == 2) { const float p = fmaxf(v, 0.f); return p * p; }
    if (act == 3) return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
    return v;
}

// x[r, c] = act(x[r, c] + bias[c]) in place (bias float or null). Rows whose size and address allow it go in
// 16-byte pieces (VEC elements a thread), anything else element by element.
template <typename T, int VEC>
__global__ void bias_act_kernel(T* __restrict__ x, const float* __restrict__ bias, long n, int width, int act) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * VEC; i < n; i += (long)gridDim.x * blockDim.x * VEC) {
        if (VEC == 1) {
            const float b = bias ? bias[i % width] : 0.f;
            x[i] = from_f32<T>(apply_act(to_f32(x[i]) + b, act));
        } else {
            const int c0 = (int)(i % width);
            union { uint4 raw; T e[VEC]; } v;
            v.raw = *reinterpret_cast<const uint4*>(x + i);
#pragma unroll
            for (int k = 0; k < VEC; ++k) v.e[k] = from_f32<T>(apply_act(to_f32(v.e[k]) + (bias ? bias[c0 + k] : 0.f), act));
            *reinterpret_cast<uint4*>(x + i) = v.raw;
        }
    }
}

extern "C" int cml_bias_act(void* x, int dtype, const float* bias, int rows, int width, int act, void* stream) {
    const long n = (long)rows * width;
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = dtype == CML_DTYPE_F32 ? 4 : 8;
    const bool wide = width % vec == 0 && ((uintptr_t)x & 15) == 0;
    const long items = wide ? n / vec : n;
    const int grid = (int)((items + 255) / 256 < 16384 ? (items + 255) / 256 : 16384);
    if (dtype == CML_DTYPE_F32) {
        if (wide) launch_pdl(bias_act_kernel<float, 4>, dim3(grid), dim3(256), 0, s, (float*)x, bias, n, width, act);
        else launch_pdl(bias_act_kernel<float, 1>, dim3(grid), dim3(256), 0, s, (float*)x, bias, n, width, act);
    } else if (dtype == CML_DTYPE_BF16) {
        if (wide) launch_pdl(bias_act_kernel<bf16, 8>, dim3(grid), dim3(256), 0, s, (bf16*)x, bias, n, width, act);
        else launch_pdl(bias_act_kernel<bf16, 1>, dim3(grid), dim3(256), 0, s, (bf16*)x, bias, n, width, act);
    } else return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// out[i] = act(sum over splits of part[split][i] + bias[column]) in the compute type: the split sums of a product
// of few rows, added in split order, then the bias (float [width] or null), then the activation (codes above).
template <typename T>
__global__ void act_from_partials_kernel(const float* __restrict__ part, int n_splits, size_t stride, T* __restrict__ out,
                                         long n, int act, const float* __restrict__ bias, int width) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float tv = part[(size_t)min(s0 + k, n_splits - 1) * stride + i];
                t[k] = s0 + k < n_splits ? tv : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) v += t[k];
        }
        if (bias) v += bias[i % width];
        out[i] = from_f32<T>(apply_act(v, act));
    }
}

extern "C" int cml_act_from_partials(const float* part, int n_splits, long stride, void* out, int dtype, long n, int act,
                                     const float* bias, int width, void* stream) {
    if (n <= 0) return 0;
    if (n_splits < 1) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    if (dtype == CML_DTYPE_F32)
        launch_pdl(act_from_partials_kernel<float>, dim3(grid), dim3(256), 0, s, part, n_splits, (size_t)stride, (float*)out, n, act, bias, width);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(act_from_partials_kernel<bf16>, dim3(grid), dim3(256), 0, s, part, n_splits, (size_t)stride, (bf16*)out, n, act, bias, width);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// x[r, c] *= sigmoid(gate[r, gate_col + c]) in place (x in the compute type, gate float).
template <typename T>
__global__ void gate_rows_kernel(T* __restrict__ x, const float* __restrict__ gate, long ldg, int gate_col, long n, int width) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long r = i / width;
        const int c = (int)(i - r * width);
        const float g = gate[r * ldg + gate_col + c];
        x[i] = from_f32<T>(to_f32(x[i]) / (1.0f + expf(-g)));
    }
}

extern "C" int cml_gate_rows(void* x, int dtype, const float* gate, long ldg, int gate_col, int rows, int width, void* stream) {
    if (rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long n = (long)rows * width;
    const int grid = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    if (dtype == CML_DTYPE_F32) launch_pdl(gate_rows_kernel<float>, dim3(grid), dim3(256), 0, s, (float*)x, gate, ldg, gate_col, n, width);
    else if (dtype == CML_DTYPE_BF16) launch_pdl(gate_rows_kernel<bf16>, dim3(grid), dim3(256), 0, s, (bf16*)x, gate, ldg, gate_col, n, width);
    else return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// x = cap * tanh(x / cap) in place (float logits).
__global__ void softcap_kernel(float* __restrict__ x, long n, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int cml_softcap(float* x, long n, float cap, void* stream) {
    if (n <= 0) return 0;
    const int grid = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    launch_pdl(softcap_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, x, n, cap);
    return cml_launch_status();
}

// x *= factor in place (float logits).
__global__ void scale_values_kernel(float* __restrict__ x, long n, float factor) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) x[i] *= factor;
}

extern "C" int cml_scale_values(float* x, long n, float factor, void* stream) {
    if (n <= 0) return 0;
    const int grid = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    launch_pdl(scale_values_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, x, n, factor);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// residual[r] += coef * sum over branches b of rmsnorm(y_b[r] + bias_b) * w_b. Each y_b is a float
// matrix [splits_b, rows, hidden] whose splits are summed first, in index order. One block
// per row; the rows of all branches are kept in shared memory between the two passes.
struct CombineBranches {
    const float* y[4];
    const void* w[4];
    const float* bias[4];       // added to the branch's summed row before its norm (null: none)
    int splits[4];
    long split_stride[4];
    int n;
};

template <typename TW>
__global__ void __launch_bounds__(512) norm_combine_kernel(CombineBranches br, float* __restrict__ residual, int hidden, float eps, float coef) {
    __shared__ float red[33];
    extern __shared__ float rowbuf[];                  // [branch][hidden]: each branch's row with its splits added
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * hidden;
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        // sixteen splits of every branch at a time: the loads are unconditional (of a valid place) and all in
        // flight before the first add; the adds stay in split order
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        int most = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) most = max(most, b < br.n ? br.splits[b] : 0);
        if (most == 1) {                               // whole rows (prompts): one load per branch
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (b < br.n) v[b] = br.y[b][(size_t)r * hidden + c];
        }
        for (int s0 = 0; most > 1 && s0 < most; s0 += 16) {
            float t[4][16];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (b >= br.n) continue;
                const float* y = br.y[b] + (size_t)r * hidden + c;
                const int ns = br.splits[b];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float tv = y[(size_t)min(s0 + i, ns - 1) * br.split_stride[b]];
                    t[b][i] = s0 + i < ns ? tv : 0.f;
                }
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (b >= br.n) continue;
#pragma unroll
                for (int i = 0; i < 16; ++i) v[b] += t[b][i];
            }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if (b >= br.n) continue;
            if (br.bias[b]) v[b] += br.bias[b][c];
            rowbuf[(size_t)b * hidden + c] = v[b];
            ss[b] = fmaf(v[b], v[b], ss[b]);
        }
    }
    float scale[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        if (b >= br.n) continue;
        scale[b] = coef / sqrtf(block_sum(ss[b], red) / (float)hidden + eps);
        __syncthreads();
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float acc = res[c];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if (b >= br.n) continue;
            acc += rowbuf[(size_t)b * hidden + c] * scale[b] * to_f32(((const TW*)br.w[b])[c]);
        }
        res[c] = acc;
    }
}

extern "C" int cml_norm_combine(const float* const* y, const void* const* w, const float* const* bias, const int* splits,
                                const long* split_stride, int n_branches, int w_dtype, float* residual, int rows, int hidden, float eps, float coef,
                                void* stream) {
    if (rows <= 0) return 0;
    if (n_branches < 1 || n_branches > 4) return CML_ERR_BAD_SIZE;
    CombineBranches br;
    br.n = n_branches;
    for (int b = 0; b < 4; ++b) {
        br.y[b] = b < n_branches ? y[b] : nullptr;
        br.w[b] = b < n_branches ? w[b] : nullptr;
        br.bias[b] = (b < n_branches && bias) ? bias[b] : nullptr;
        br.splits[b] = b < n_branches ? splits[b] : 0;
        br.split_stride[b] = b < n_branches ? split_stride[b] : 0;
    }
    cudaStream_t s = (cudaStream_t)stream;
    // few rows (one-token steps): many threads per row shorten each thread's chain of columns
    int block = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (rows <= 256 && hidden >= 1024) block = 512;
    else if (block > 256) block = 256;               // many rows: several blocks per SM
    const size_t smem = (size_t)n_branches * hidden * sizeof(float);
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
    if (w_dtype == CML_DTYPE_F32) {
        if (smem > 48 * 1024 && cml_allow_smem<norm_combine_kernel<float>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE;
        launch_pdl(norm_combine_kernel<float>, dim3(rows), dim3(block), smem, s, br, residual, hidden, eps, coef);
    } else if (w_dtype == CML_DTYPE_BF16) {
        if (smem > 48 * 1024 && cml_allow_smem<norm_combine_kernel<bf16>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE;
        launch_pdl(norm_combine_kernel<bf16>, dim3(rows), dim3(block), smem, s, br, residual, hidden, eps, coef);
    } else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// The norm behind a sublayer and, where wanted, the norm before the next one, in one pass over a row:
//   v = sum over splits of y[split][r] + bias;   h[r] += coef * v / sqrt(mean(v^2) + eps) * w_post;
//   x_out[r] = h[r] / sqrt(mean(h[r]^2) + eps_next) * w_next     (if x_out is given)
//   (x_out given without w_next: x_out[r] = h[r] in the compute type)
// One block per row; the row stays in shared memory between the passes; all sums in float.
template <typename TW, typename TO>
__global__ void __launch_bounds__(512) post_norm_add_kernel(const float* __restrict__ y, int n_splits, long split_stride,
                                                            const float* __restrict__ bias, const TW* __restrict__ w_post,
                                                            float eps, float coef, float* __restrict__ h,
                                                            const TW* __restrict__ w_next, float eps_next,
                                                            TO* __restrict__ x_out, int hidden) {
    extern __shared__ __align__(16) float pn_row[];
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t base = (size_t)blockIdx.x * hidden;
    const bool vec = (hidden & 3) == 0;
    float ss = 0.f;
    if (vec) {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(y + base + c);
            // the other splits eight at a time: unconditional loads (of a valid place), all in flight before the first
            // add; the adds stay in split order
            for (int s0 = 1; s0 < n_splits; s0 += 8) {
                float4 t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    t[k] = *reinterpret_cast<const float4*>(y + (size_t)min(s0 + k, n_splits - 1) * split_stride + base + c);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < n_splits) { v.x += t[k].x; v.y += t[k].y; v.z += t[k].z; v.w += t[k].w; }
            }
            if (bias) { v.x += bias[c]; v.y += bias[c + 1]; v.z += bias[c + 2]; v.w += bias[c + 3]; }
            *reinterpret_cast<float4*>(pn_row + c) = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            float v = y[base + c];
            for (int s = 1; s < n_splits; ++s) v += y[(size_t)s * split_stride + base + c];
            if (bias) v += bias[c];
            pn_row[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    const float s1 = coef / sqrtf(block_sum(ss, red) / (float)hidden + eps);
    __syncthreads();
    float ss2 = 0.f;
    if (vec) {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(pn_row + c);
            float4 o = *reinterpret_cast<const float4*>(h + base + c);
            o.x += v.x * s1 * to_f32(w_post[c]); o.y += v.y * s1 * to_f32(w_post[c + 1]);
            o.z += v.z * s1 * to_f32(w_post[c + 2]); o.w += v.w * s1 * to_f32(w_post[c + 3]);
            *reinterpret_cast<float4*>(h + base + c) = o;
            *reinterpret_cast<float4*>(pn_row + c) = o;
            ss2 = fmaf(o.x, o.x, fmaf(o.y, o.y, fmaf(o.z, o.z, fmaf(o.w, o.w, ss2))));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float o = h[base + c] + pn_row[c] * s1 * to_f32(w_post[c]);
            h[base + c] = o;
            pn_row[c] = o;
            ss2 = fmaf(o, o, ss2);
        }
    }
    if (x_out == nullptr) return;
    const float s2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)hidden + eps_next);
    if (w_next == nullptr) {                                      // no norm before the next reader: the stream's rows themselves
        if (!vec) {
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) x_out[base + c] = from_f32<TO>(pn_row[c]);
        } else {
            for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
                const float4 o = *reinterpret_cast<const float4*>(pn_row + c);
                x_out[base + c] = from_f32<TO>(o.x); x_out[base + c + 1] = from_f32<TO>(o.y);
                x_out[base + c + 2] = from_f32<TO>(o.z); x_out[base + c + 3] = from_f32<TO>(o.w);
            }
        }
        return;
    }
    if (!vec) {                                                   // each thread reads back what it wrote itself
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) x_out[base + c] = from_f32<TO>(pn_row[c] * s2 * to_f32(w_next[c]));
    } else {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            const float4 o = *reinterpret_cast<const float4*>(pn_row + c);
            x_out[base + c] = from_f32<TO>(o.x * s2 * to_f32(w_next[c]));
            x_out[base + c + 1] = from_f32<TO>(o.y * s2 * to_f32(w_next[c + 1]));
            x_out[base + c + 2] = from_f32<TO>(o.z * s2 * to_f32(w_next[c + 2]));
            x_out[base + c + 3] = from_f32<TO>(o.w * s2 * to_f32(w_next[c + 3]));
        }
    }
}

extern "C" int cml_post_norm_add(const float* y, int n_splits, long split_stride, const float* bias, const void* w_post, int w_dtype,
                                 float eps, float coef, float* h, const void* w_next, float eps_next, void* x_out, int out_dtype,
                                 int rows, int hidden, void* stream) {
    if (rows <= 0) return 0;
    if (n_splits < 1) return CML_ERR_BAD_SIZE;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    // few rows (one-token steps): more threads per row shorten each thread's chain of columns
    const int block = rows <= 256 && hidden >= 2048 ? 512 : (hidden >= 1024 ? 256 : 128);
#define PN_CASE(TW_, TO_, DW_, DO_)                                                                                        \
    if (w_dtype == DW_ && (x_out == nullptr || out_dtype == DO_)) {                                                        \
        if (smem > 48 * 1024 && cml_allow_smem<post_norm_add_kernel<TW_, TO_>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE; \
        launch_pdl(post_norm_add_kernel<TW_, TO_>, dim3(rows), dim3(block), smem, s, y, n_splits, split_stride, bias,     \
                   (const TW_*)w_post, eps, coef, h, (const TW_*)w_next, eps_next, (TO_*)x_out, hidden);                   \
        return cml_launch_status();                                                                                        \
    }
    PN_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    PN_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    PN_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
    PN_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
#undef PN_CASE
    return CML_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------
// The norm *after* a residual sum, where the stream itself is normed (no separate sum is kept):
//   v = alpha * h[r] + sum over splits of y[split][r] + bias;   h[r] = v / sqrt(mean(v^2) + eps) * w
// and, where x_out is given, the same row in the compute type for the products that read the stream next.
// One block per row; the row stays in shared memory between the passes; all sums in float.
template <typename TW, typename TO>
__global__ void __launch_bounds__(512) sum_norm_kernel(const float* __restrict__ y, int n_splits, long split_stride,
                                                       const float* __restrict__ bias, const TW* __restrict__ w, float eps,
                                                       float alpha, float* __restrict__ h, TO* __restrict__ x_out, int hidden) {
    extern __shared__ __align__(16) float sn_row[];
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t base = (size_t)blockIdx.x * hidden;
    const bool vec = (hidden & 3) == 0;
    float ss = 0.f;
    if (vec) {
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(y + base + c);
            const float4 o = *reinterpret_cast<const float4*>(h + base + c);
            for (int s0 = 1; s0 < n_splits; s0 += 8) {          // eight splits' loads in flight; the adds stay in split order
                float4 t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    t[k] = *reinterpret_cast<const float4*>(y + (size_t)min(s0 + k, n_splits - 1) * split_stride + base + c);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < n_splits) { v.x += t[k].x; v.y += t[k].y; v.z += t[k].z; v.w += t[k].w; }
            }
            if (bias) { v.x += bias[c]; v.y += bias[c + 1]; v.z += bias[c + 2]; v.w += bias[c + 3]; }
            v.x = fmaf(alpha, o.x, v.x); v.y = fmaf(alpha, o.y, v.y); v.z = fmaf(alpha, o.z, v.z); v.w = fmaf(alpha, o.w, v.w);
            *reinterpret_cast<float4*>(sn_row + c) = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            float v = y[base + c];
            for (int s = 1; s < n_splits; ++s) v += y[(size_t)s * split_stride + base + c];
            if (bias) v += bias[c];
            v = fmaf(alpha, h[base + c], v);
            sn_row[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    const float sc = 1.0f / sqrtf(block_sum(ss, red) / (float)hidden + eps);
    if (vec) {                                                    // each thread reads back what it wrote itself
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(sn_row + c);
            const float4 o = make_float4(v.x * sc * to_f32(w[c]), v.y * sc * to_f32(w[c + 1]), v.z * sc * to_f32(w[c + 2]),
                                         v.w * sc * to_f32(w[c + 3]));
            *reinterpret_cast<float4*>(h + base + c) = o;
            if (x_out) {
                x_out[base + c] = from_f32<TO>(o.x); x_out[base + c + 1] = from_f32<TO>(o.y);
                x_out[base + c + 2] = from_f32<TO>(o.z); x_out[base + c + 3] = from_f32<TO>(o.w);
            }
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float o = sn_row[c] * sc * to_f32(w[c]);
            h[base + c] = o;
            if (x_out) x_out[base + c] = from_f32<TO>(o);
        }
    }
}

extern "C" int cml_sum_norm(const float* y, int n_splits, long split_stride, const float* bias, const void* w, int w_dtype, float eps,
                            float alpha, float* h, void* x_out, int out_dtype, int rows, int hidden, void* stream) {
    if (rows <= 0) return 0;
    if (n_splits < 1) return CML_ERR_BAD_SIZE;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = rows <= 256 && hidden >= 2048 ? 512 : (hidden >= 1024 ? 256 : 128);
#define SN_CASE(TW_, TO_, DW_, DO_)                                                                                        \
    if (w_dtype == DW_ && (x_out == nullptr || out_dtype == DO_)) {                                                        \
        if (smem > 48 * 1024 && cml_allow_smem<sum_norm_kernel<TW_, TO_>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE;    \
        launch_pdl(sum_norm_kernel<TW_, TO_>, dim3(rows), dim3(block), smem, s, y, n_splits, split_stride, bias,          \
                   (const TW_*)w, eps, alpha, h, (TO_*)x_out, hidden);                                                     \
        return cml_launch_status();                                                                                        \
    }
    SN_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    SN_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    SN_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
    SN_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
#undef SN_CASE
    return CML_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------
// out[r, c] = gelu_tanh(sum over splits of z[split][r, c]) * table[tokens[r], col0 + c] in the compute type: the gate of
// a per-layer token input, times the layer's own columns of a second embedding table. One thread per element.
template <typename T>
__global__ void gelu_mul_lookup_kernel(const float* __restrict__ z, long ldz, int n_splits, long split_stride,
                                       const T* __restrict__ table, long ldt, int col0, const int* __restrict__ tokens,
                                       int vocab, T* __restrict__ out, int rows, int dim) {
    pdl_wait();
    pdl_launch_dependents();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)rows * dim) return;
    const int r = (int)(i / dim), c = (int)(i % dim);
    float v = z[(size_t)r * ldz + c];
    for (int s = 1; s < n_splits; ++s) v += z[(size_t)s * split_stride + (size_t)r * ldz + c];
    const int tok = min(max(tokens[r], 0), vocab - 1);          // ids are checked on the host and by the embedding kernel
    out[i] = from_f32<T>(gelu_tanh_f(v) * to_f32(table[(size_t)tok * ldt + col0 + c]));
}

extern "C" int cml_gelu_mul_lookup(const float* z, long ldz, int n_splits, long split_stride, const void* table, int dtype, long ldt,
                                   int col0, const int* tokens, int vocab, void* out, int rows, int dim, void* stream) {
    if (rows <= 0 || dim <= 0) return 0;
    if (n_splits < 1) return CML_ERR_BAD_SIZE;
    const long n = (long)rows * dim;
    const dim3 grid((unsigned)((n + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(gelu_mul_lookup_kernel<float>, grid, dim3(256), 0, s, z, ldz, n_splits, split_stride, (const float*)table, ldt, col0,
                   tokens, vocab, (float*)out, rows, dim);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(gelu_mul_lookup_kernel<bf16>, grid, dim3(256), 0, s, z, ldz, n_splits, split_stride, (const bf16*)table, ldt, col0,
                   tokens, vocab, (bf16*)out, rows, dim);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// out[i] = x[i] in the compute type: the float stream's rows for products that read the stream as it is.
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) out[i] = from_f32<T>(x[i]);
}

extern "C" int cml_cast_rows(const float* x, void* out, int dtype, long n, void* stream) {
    if (n <= 0) return 0;
    const long blocks = (n + 255) / 256;
    const dim3 grid((unsigned)(blocks < 4096 ? blocks : 4096));
    if (dtype == CML_DTYPE_F32) launch_pdl(cast_rows_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, x, (float*)out, n);
    else if (dtype == CML_DTYPE_BF16) launch_pdl(cast_rows_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, x, (bf16*)out, n);
    else return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
