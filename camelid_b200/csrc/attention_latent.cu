// Attention over a latent: every position keeps one normed row c of C channels (from which all heads' keys and values
// are linear maps, k_h = Uk_h c, v_h = Uv_h c) and one turned key part of R channels that all heads share. The maps are
// moved to the query's side: with q_h = [a_h (D channels), b_h (R, turned)],
//
//   score_h(i, j) = (a_h . Uk_h c_j + b_h . t_j) scale = ([Uk_h^T a_h, b_h] . [c_j, t_j]) scale
//   out_h(i)      = Uv_h (sum_j w_ij c_j)
//
// so the cache holds rows [c_j, t_j] of C + R channels, one "key head" for all query heads, whose first C channels are
// the values as well; the attention itself is the library's general kernel (attention_window.cu). Here: the kernel that
// prepares a step's rows, and the product per head that applies Uk_h^T to the queries and Uv_h to the outputs.
#include "common.cuh"

// proj [rows, ld] float (n_splits matrices split_stride apart, added in split order): q (heads x (D + R), head by head
// [plain D, turned R]), then C + R columns of the down projection, then `extra` columns (an output gate's logits).
// One block per row:
//   q_plain [rows, heads x D]           the unturned query parts, compute type
//   q_full  [rows, heads x (C + R)]     the turned parts, at channels C.. of every head (the first C are written later)
//   k_pages [pages, 1, 64, C + R]       [rmsnorm(down[:C]) * w, turned(down[C:])]
//   extra_out [rows, extra]             float
// Turning: angle = position * inv_freq[i], sines and cosines times amp, pairs (2i, 2i + 1) (pairing 1) or (i, i + R / 2).
template <typename T, typename TW>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const float* __restrict__ proj, long ld, int n_splits, long split_stride,
                                                             int extra, float* __restrict__ extra_out, const TW* __restrict__ c_w, float eps,
                                                             const float* __restrict__ inv_freq, int pairing, float amp,
                                                             const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                                             const int* __restrict__ table, int max_blocks, T* __restrict__ q_plain,
                                                             T* __restrict__ q_full, T* __restrict__ k_pages, int heads, int D, int R, int C) {
    __shared__ float red[32];
    __shared__ float2 turn[128];
    extern __shared__ __align__(16) float x[];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int qw = heads * (D + R), total = qw + C + R + extra;
    const float* src = proj + (size_t)r * ld;
    float ss = 0.f;
    for (int c = threadIdx.x; c < total; c += blockDim.x) {
        float v = src[c];
        for (int s0 = 1; s0 < n_splits; s0 += 8) {
            float t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = src[(size_t)min(s0 + k, n_splits - 1) * split_stride + c];
#pragma unroll
            for (int k = 0; k < 8; ++k) v += s0 + k < n_splits ? t[k] : 0.f;
        }
        x[c] = v;
        if (c >= qw && c < qw + C) ss = fmaf(v, v, ss);
    }
    const int pos = row_pos[r];
    const int page = table[(size_t)row_seq[r] * max_blocks + pos / CML_PAGE];
    for (int i = threadIdx.x; i < R / 2; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        turn[i] = make_float2(cs * amp, sn * amp);
    }
    const float c_scale = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);       // (has the barrier that x and turn need)
    for (int c = threadIdx.x; c < extra; c += blockDim.x) extra_out[(size_t)r * extra + c] = x[total - extra + c];
    const int half = R / 2;
    // channel e of a turned part that starts at xs
    auto turned = [&](const float* xs, int e) -> float {
        const bool first = pairing ? !(e & 1) : e < half;
        const int other = pairing ? (first ? e + 1 : e - 1) : (first ? e + half : e - half);
        const float2 t = turn[pairing ? e >> 1 : (first ? e : e - half)];
        return first ? xs[e] * t.x - xs[other] * t.y : xs[e] * t.x + xs[other] * t.y;
    };
    for (int c = threadIdx.x; c < heads * D; c += blockDim.x) {
        const int hd = c / D, e = c - hd * D;
        q_plain[(size_t)r * heads * D + c] = from_f32<T>(x[hd * (D + R) + e]);
    }
    for (int c = threadIdx.x; c < heads * R; c += blockDim.x) {
        const int hd = c / R, e = c - hd * R;
        q_full[((size_t)r * heads + hd) * (C + R) + C + e] = from_f32<T>(turned(x + hd * (D + R) + D, e));
    }
    if (page >= 0) {
        T* k_row = k_pages + ((size_t)page * CML_PAGE + pos % CML_PAGE) * (C + R);
        for (int c = threadIdx.x; c < C; c += blockDim.x) k_row[c] = from_f32<T>(x[qw + c] * c_scale * to_f32(c_w[c]));
        for (int e = threadIdx.x; e < R; e += blockDim.x) k_row[C + e] = from_f32<T>(turned(x + qw + C, e));
    }
}

extern "C" int cml_latent_prepare(const float* proj, long ld, int n_splits, long split_stride, int extra, float* extra_out,
                                  const void* c_w, int w_dtype, float eps, const float* inv_freq, int pairing, float amp,
                                  const int* row_seq, const int* row_pos, const int* table, int max_blocks, void* q_plain,
                                  void* q_full, void* k_pages, int dtype, int rows, int heads, int D, int R, int C, void* stream) {
    if (rows <= 0) return 0;
    if (R < 0 || R > 256 || (R & 1) || C < 1 || D < 0 || n_splits < 1 || extra < 0) return CML_ERR_BAD_SIZE;
    const size_t smem = (size_t)(heads * (D + R) + C + R + extra + 4) * sizeof(float);
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
#define LP_CASE(T_, TW_, D_, DW_)                                                                                               \
    if (dtype == D_ && w_dtype == DW_) {                                                                                        \
        if (smem > 48 * 1024 && cml_allow_smem<latent_prepare_kernel<T_, TW_>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE;   \
        launch_pdl(latent_prepare_kernel<T_, TW_>, dim3(rows), dim3(256), smem, s, proj, ld, n_splits, split_stride, extra,     \
                   extra_out, (const TW_*)c_w, eps, inv_freq, pairing, amp, row_seq, row_pos, table, max_blocks, (T_*)q_plain,  \
                   (T_*)q_full, (T_*)k_pages, heads, D, R, C);                                                                  \
        return cml_launch_status();                                                                                             \
    }
    LP_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    LP_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    LP_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    LP_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
#undef LP_CASE
    return CML_ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------------
// A product per head: out[r, h, n] = sum_k x[r, h, k] * w[h, n, k], float accumulation, k in order.
// x [rows, ldx] with head h at column h * xs; w [heads, N, K] contiguous; out [rows, ldo] with head h at column h * os.
// A block owns HP_ROWS rows x HP_COLS outputs of one head; K passes through shared memory HP_K channels at a time
// (weights transposed on the way in, rows padded against bank conflicts); a thread keeps 2 x 4 sums.
#define HP_ROWS 32
#define HP_COLS 64
#define HP_K 32

template <typename T>
__global__ void __launch_bounds__(256) head_product_kernel(const T* __restrict__ x, long ldx, int xs, const T* __restrict__ w,
                                                           T* __restrict__ out, long ldo, int os, int rows, int N, int K) {
    __shared__ float sx[HP_ROWS][HP_K + 1];
    __shared__ float sw[HP_K][HP_COLS + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int hd = blockIdx.z, r0 = blockIdx.y * HP_ROWS, n0 = blockIdx.x * HP_COLS;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 16 x 16 threads: columns tx + 16 j, rows ty + 16 i
    const T* wh = w + (size_t)hd * N * K;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += HP_K) {
        for (int i = threadIdx.x; i < HP_ROWS * HP_K; i += 256) {
            const int rr = i / HP_K, kk = i % HP_K;
            const bool ok = r0 + rr < rows && k0 + kk < K;
            sx[rr][kk] = ok ? to_f32(x[(size_t)(r0 + rr) * ldx + (size_t)hd * xs + k0 + kk]) : 0.f;
        }
        for (int i = threadIdx.x; i < HP_COLS * HP_K; i += 256) {
            const int nn = i / HP_K, kk = i % HP_K;
            const bool ok = n0 + nn < N && k0 + kk < K;
            sw[kk][nn] = ok ? to_f32(wh[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < HP_K; ++kk) {
            const float a0 = sx[ty][kk], a1 = sx[ty + 16][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = sw[kk][tx + 16 * j];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rr = r0 + ty + 16 * i;
        if (rr >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nn = n0 + tx + 16 * j;
            if (nn < N) out[(size_t)rr * ldo + (size_t)hd * os + nn] = from_f32<T>(acc[i][j]);
        }
    }
}

extern "C" int cml_head_product(const void* x, long ldx, int xs, const void* w, void* out, long ldo, int os, int dtype, int rows,
                                int heads, int N, int K, void* stream) {
    if (rows <= 0 || heads <= 0 || N <= 0) return 0;
    if (K < 1 || heads > 65535 || (rows + HP_ROWS - 1) / HP_ROWS > 65535) return CML_ERR_BAD_SIZE;
    dim3 grid((unsigned)((N + HP_COLS - 1) / HP_COLS), (unsigned)((rows + HP_ROWS - 1) / HP_ROWS), (unsigned)heads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(head_product_kernel<float>, grid, dim3(256), 0, s, (const float*)x, ldx, xs, (const float*)w, (float*)out, ldo, os,
                   rows, N, K);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(head_product_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)x, ldx, xs, (const bf16*)w, (bf16*)out, ldo, os,
                   rows, N, K);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
