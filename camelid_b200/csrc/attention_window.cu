// Softmax attention over a sliding window of the paged cache, without rotation, for mixers
// whose keys and values may differ in size: per-head RMS norm of q and k, a penalty on the
// distance between query and key, an output gate.
//
//   score(i, j) = (q_i . k_j) scale - r1[head] ln(1 + r2[head] (i - j)),   0 <= i - j < window
//
// Besides the window, a query may be held to the keys of its own block of `chunk` positions (blocks
// counted from position 0 of the sequence); the softmax denominator may hold one more term
// exp(sink[head]) that has no key and no value; the gate may be one number per head. A second
// preparing kernel normalises q and k over their whole projections (all heads at once) and rotates
// pairs of channels by the position (pairs of neighbours, or of the two halves of the rotated part).
//
// Two kernels. The first normalises q and k (weight per channel, shared by the heads), keeps
// q in the compute type and writes k and v into their pages. The second gives a block to
// every (row, head): lanes take keys for the scores (all in float), then columns of the
// values; the softmax runs online over rounds of 32 keys, from the oldest visible key to the
// row's own, whether the row came with a prompt or alone. With `keep_first` > 0 the first keep_first keys of the
// sequence stay visible beside the window; they come first in the order of the rounds. `v_stride`: channels between two
// value rows of a page (Dv; or the key rows' size where the values are the first Dv channels of the key rows themselves).
#include "common.cuh"

__device__ __forceinline__ float sigmoid_w(float x) { return 1.0f / (1.0f + expf(-x)); }

// proj [rows, ld] float: q (heads x D) at column 0, k (kv_heads x D), v (kv_heads x Dv).
// q_out [rows, heads x D]; pages [pages, kv_heads, 64, D | Dv]; table [seqs, max_blocks].
// With maps > 1 every q and k head holds `maps` score maps of D channels side by side (D = head size / maps), each
// normed on its own with the same weight of D channels; the cache keeps a key head's maps as one row of maps x D.
template <typename T, typename TW>
__global__ void qk_norm_kv_write_kernel(const float* __restrict__ proj, long ld, const TW* __restrict__ q_w,
                                        const TW* __restrict__ k_w, int qk_norm, float eps, const int* __restrict__ row_seq,
                                        const int* __restrict__ row_pos, const int* __restrict__ table, int max_blocks,
                                        T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int rows,
                                        int heads, int kv_heads_all, int D, int Dv, int maps) {
    pdl_wait();
    pdl_launch_dependents();
    // units: a query map, a key map, a value head; `heads` and `kv_heads` below count maps
    const int v_heads = kv_heads_all, kv_heads = kv_heads_all * maps;
    heads *= maps;
    const int units = heads + kv_heads + v_heads;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * units) return;
    const int r = warp / units, u = warp % units;
    const float* x = proj + (size_t)r * ld;
    if (u < heads) {                                            // a query head
        x += u * D;
        float scale = 1.0f;
        if (qk_norm) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(x[c], x[c], ss);
            scale = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        T* o = q_out + ((size_t)r * heads + u) * D;
        for (int c = lane; c < D; c += 32) o[c] = from_f32<T>(qk_norm ? x[c] * scale * to_f32(q_w[c]) : x[c]);
        return;
    }
    const int pos = row_pos[r];
    const int page = table[(size_t)row_seq[r] * max_blocks + pos / CML_PAGE];
    if (page < 0) return;                                       // never for a row of the step
    if (u < heads + kv_heads) {                                 // a key head
        const int g = u - heads;
        x += heads * D + g * D;
        float scale = 1.0f;
        if (qk_norm) {
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(x[c], x[c], ss);
            scale = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        T* o = k_pages + ((((size_t)page * v_heads + g / maps) * CML_PAGE + pos % CML_PAGE) * maps + g % maps) * D;
        for (int c = lane; c < D; c += 32) o[c] = from_f32<T>(qk_norm ? x[c] * scale * to_f32(k_w[c]) : x[c]);
    } else {                                                    // a value head
        const int g = u - heads - kv_heads;
        x += (heads + kv_heads) * D + g * Dv;
        T* o = v_pages + (((size_t)page * v_heads + g) * CML_PAGE + pos % CML_PAGE) * Dv;
        for (int c = lane; c < Dv; c += 32) o[c] = from_f32<T>(x[c]);
    }
}

extern "C" int cml_qk_norm_kv_write(const float* proj, long ld, const void* q_w, const void* k_w, int w_dtype, int qk_norm,
                                    float eps, const int* row_seq, const int* row_pos, const int* table, int max_blocks,
                                    void* q_out, void* k_pages, void* v_pages, int dtype, int rows, int heads, int kv_heads,
                                    int D, int Dv, int maps, void* stream) {
    if (rows <= 0) return 0;
    if (maps < 1) return CML_ERR_BAD_SIZE;
    const long warps = (long)rows * (maps * (heads + kv_heads) + kv_heads);
    dim3 grid((unsigned)((warps + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
#define QK_CASE(T_, TW_, D_, DW_)                                                                                          \
    if (dtype == D_ && w_dtype == DW_) {                                                                                   \
        launch_pdl(qk_norm_kv_write_kernel<T_, TW_>, grid, dim3(128), 0, s, proj, ld, (const TW_*)q_w, (const TW_*)k_w, qk_norm, \
                   eps, row_seq, row_pos, table, max_blocks, (T_*)q_out, (T_*)k_pages, (T_*)v_pages, rows, heads, kv_heads, D, \
                   Dv, maps);                                                                                                    \
        return cml_launch_status();                                                                                        \
    }
    QK_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    QK_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    QK_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    QK_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
#undef QK_CASE
    return CML_ERR_BAD_DTYPE;
}

// The same job for mixers that rotate: proj [rows, ld] float holds q, k, v as above. norm_mode 0: q and k as
// they are; 1: RMS norm per head, weights of D channels shared by the heads; 2: RMS norm over the whole q
// projection (heads x D channels at once) and the whole k projection, weights of those sizes. Then the first
// rot_dim channels of every q and k head are rotated by angle = position * inv_freq[i] (float), pairing 1:
// channels (2i, 2i + 1); pairing 0: channels (i, i + rot_dim / 2). One block per row. proj may come as split sums
// (n_splits matrices split_stride apart, added here in split order); the row is staged in shared memory, its sums
// of squares taken on the way in. `extra` more columns behind v (the logits of an output gate) are copied, summed,
// to extra_out [rows, extra]. `bias` (float, q, k, v and the extra columns; or null) is added to the summed row before
// the norms; `rot_amp` multiplies every sine and cosine. A warp works on one head at a time, a lane on four neighbouring channels (two, or
// one, where the head size allows no more), so that a warp's stores are one contiguous run.
template <typename T> __device__ __forceinline__ void store_run(T* o, const float* v, int n);
template <> __device__ __forceinline__ void store_run<float>(float* o, const float* v, int n) {
    if (n == 4) *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
    else if (n == 2) *reinterpret_cast<float2*>(o) = make_float2(v[0], v[1]);
    else o[0] = v[0];
}
template <> __device__ __forceinline__ void store_run<bf16>(bf16* o, const float* v, int n) {
    if (n == 4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else if (n == 2) {
        *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(v[0], v[1]);
    } else {
        o[0] = __float2bfloat16_rn(v[0]);
    }
}

template <typename T, typename TW, int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS <= 256 ? 5 : 1)
qkv_prepare_kernel(const float* __restrict__ proj, long ld, int n_splits, long split_stride, int extra,
                   float* __restrict__ extra_out, const TW* __restrict__ q_w, const TW* __restrict__ k_w, int norm_mode, float eps,
                   const float* __restrict__ inv_freq, int rot_dim, int pairing, const int* __restrict__ row_seq,
                   const int* __restrict__ row_pos, const int* __restrict__ table, int max_blocks, T* __restrict__ q_out,
                   T* __restrict__ k_pages, T* __restrict__ v_pages, int heads, int kv_heads, int D, int Dv,
                   const float* __restrict__ bias, float rot_amp) {
    __shared__ float red[2][32];
    __shared__ float2 turn[128];                                // (cosine, sine) of the row's angles, shared by all heads
    extern __shared__ __align__(16) float x[];                 // the row: q, k, v, the extra columns
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NWARPS = THREADS / 32;
    const int qw = heads * D, kw = kv_heads * D, vw = kv_heads * Dv;
    const int total = qw + kw + vw + extra;
    const float* src = proj + (size_t)r * ld;
    float sq = 0.f, sk = 0.f;                                   // sums of squares of the q and the k columns
    if (((ld | split_stride | (long)total) & 3) == 0 && (((uintptr_t)proj) & 15) == 0) {
        for (int c = threadIdx.x * 4; c < total; c += THREADS * 4) {
            float4 v = *reinterpret_cast<const float4*>(src + c);
            // the other splits eight at a time: unconditional loads (of a valid place), all in flight before the first
            // add; the adds stay in split order
            for (int s0 = 1; s0 < n_splits; s0 += 8) {
                float4 t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    t[k] = *reinterpret_cast<const float4*>(src + (size_t)min(s0 + k, n_splits - 1) * split_stride + c);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (s0 + k < n_splits) { v.x += t[k].x; v.y += t[k].y; v.z += t[k].z; v.w += t[k].w; }
            }
            if (bias != nullptr) {                              // the projections' biases, after the sums
                const float4 b = *reinterpret_cast<const float4*>(bias + c);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            *reinterpret_cast<float4*>(x + c) = v;
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (c + i < qw) sq = fmaf(e[i], e[i], sq);
                else if (c + i < qw + kw) sk = fmaf(e[i], e[i], sk);
            }
        }
    } else {
        for (int c = threadIdx.x; c < total; c += THREADS) {
            float v = src[c];
            for (int s0 = 1; s0 < n_splits; s0 += 8) {
                float t[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) t[k] = src[(size_t)min(s0 + k, n_splits - 1) * split_stride + c];
#pragma unroll
                for (int k = 0; k < 8; ++k) v += s0 + k < n_splits ? t[k] : 0.f;
            }
            if (bias != nullptr) v += bias[c];
            x[c] = v;
            if (c < qw) sq = fmaf(v, v, sq);
            else if (c < qw + kw) sk = fmaf(v, v, sk);
        }
    }
    const int pos = row_pos[r];
    const int page = table[(size_t)row_seq[r] * max_blocks + pos / CML_PAGE];
    for (int i = threadIdx.x; i < rot_dim / 2; i += THREADS) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        turn[i] = make_float2(cs * rot_amp, sn * rot_amp);
    }
    if (norm_mode == 2) {                                       // both sums over the block with one barrier
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
    }
    __syncthreads();
    float q_scale = 1.0f, k_scale = 1.0f;
    if (norm_mode == 2) {
        q_scale = 1.0f / sqrtf(warp_sum(lane < NWARPS ? red[0][lane] : 0.f) / (float)qw + eps);
        k_scale = 1.0f / sqrtf(warp_sum(lane < NWARPS ? red[1][lane] : 0.f) / (float)kw + eps);
    }
    for (int c = threadIdx.x; c < extra; c += THREADS) extra_out[(size_t)r * extra + c] = x[total - extra + c];
    const int half = rot_dim / 2;
    T* k_row = page >= 0 ? k_pages + ((size_t)page * kv_heads * CML_PAGE + pos % CML_PAGE) * D : nullptr;
    const int run = (D & 3) == 0 ? 4 : (D & 1) == 0 ? 2 : 1;     // neighbouring channels a lane takes
    for (int u = warp; u < heads + kv_heads; u += NWARPS) {
        const bool is_q = u < heads;
        const int hd = is_q ? u : u - heads;
        const float* xh = x + u * D;
        float sc = is_q ? q_scale : k_scale;
        if (norm_mode == 1) {                                   // the head's own scale
            float ss = 0.f;
            for (int c = lane; c < D; c += 32) ss = fmaf(xh[c], xh[c], ss);
            sc = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
        }
        const TW* w = (is_q ? q_w : k_w) + (norm_mode == 2 ? hd * D : 0);
        T* o = is_q ? q_out + (size_t)r * qw + hd * D : (k_row != nullptr ? k_row + (size_t)hd * CML_PAGE * D : nullptr);
        if (o == nullptr) continue;
        // channel d of the head after the norm
        auto normed = [&](int d) -> float { return norm_mode ? xh[d] * sc * to_f32(w[d]) : xh[d]; };
        for (int d = run * lane; d < D; d += run * 32) {
            float out[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = i < run ? normed(d + i) : 0.f;
            if (d < rot_dim) {
                if (pairing && run > 1) {                       // neighbours are each other's partners
#pragma unroll
                    for (int i = 0; i < 4; i += 2) {
                        if (i < run && d + i < rot_dim) {
                            const float2 t = turn[(d + i) >> 1];
                            const float a = out[i], b = out[i + 1];
                            out[i] = a * t.x - b * t.y;
                            out[i + 1] = b * t.x + a * t.y;
                        }
                    }
                } else {                                        // the partner is elsewhere in the head: fetched and normed again
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c = d + i;
                        if (i < run && c < rot_dim) {
                            const bool first = pairing ? !(c & 1) : c < half;
                            const int other = pairing ? (first ? c + 1 : c - 1) : (first ? c + half : c - half);
                            const float2 t = turn[pairing ? c >> 1 : (first ? c : c - half)];
                            const float b = normed(other);
                            out[i] = first ? out[i] * t.x - b * t.y : out[i] * t.x + b * t.y;
                        }
                    }
                }
            }
            store_run<T>(o + d, out, run);
        }
    }
    if (page >= 0) {
        T* v_row = v_pages + ((size_t)page * kv_heads * CML_PAGE + pos % CML_PAGE) * Dv;
        const float* xv = x + qw + kw;
        if ((Dv & 3) == 0 && ((qw + kw) & 3) == 0) {
            for (int c = threadIdx.x * 4; c < vw; c += THREADS * 4) {
                const int g = c / Dv, e = c - g * Dv;
                const float4 v = *reinterpret_cast<const float4*>(xv + c);
                const float vals[4] = {v.x, v.y, v.z, v.w};
                store_run<T>(v_row + (size_t)g * CML_PAGE * Dv + e, vals, 4);
            }
        } else {
            for (int c = threadIdx.x; c < vw; c += THREADS) {
                const int g = c / Dv, e = c - g * Dv;
                v_row[(size_t)g * CML_PAGE * Dv + e] = from_f32<T>(xv[c]);
            }
        }
    }
}

extern "C" int cml_qkv_prepare(const float* proj, long ld, int n_splits, long split_stride, int extra, float* extra_out,
                               const void* q_w, const void* k_w, int w_dtype, int norm_mode, float eps, const float* inv_freq,
                               int rot_dim, int pairing, const int* row_seq, const int* row_pos, const int* table,
                               int max_blocks, void* q_out, void* k_pages, void* v_pages, int dtype, int rows, int heads,
                               int kv_heads, int D, int Dv, const float* bias, float rot_amp, void* stream) {
    if (rows <= 0) return 0;
    if (rot_dim < 0 || rot_dim > D || rot_dim > 256 || (rot_dim & 1) || norm_mode < 0 || norm_mode > 2) return CML_ERR_BAD_SIZE;
    if (n_splits < 1 || extra < 0) return CML_ERR_BAD_SIZE;
    // the vector stores want aligned rows: the outputs' bases come 16-byte aligned from the allocator, the sizes decide the rest
    if ((((uintptr_t)q_out) | ((uintptr_t)k_pages) | ((uintptr_t)v_pages) | ((uintptr_t)bias)) & 15) return CML_ERR_BAD_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(heads * D + kv_heads * (D + Dv) + extra + 4) * sizeof(float);
    if (smem > 200 * 1024) return CML_ERR_BAD_SIZE;
    const bool few = rows <= 128;                               // one-token steps: more threads per row
#define QP_LAUNCH(T_, TW_, N_)                                                                                             \
    {                                                                                                                      \
        if (smem > 48 * 1024 && cml_allow_smem<qkv_prepare_kernel<T_, TW_, N_>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE; \
        launch_pdl(qkv_prepare_kernel<T_, TW_, N_>, dim3(rows), dim3(N_), smem, s, proj, ld, n_splits, split_stride, extra, \
                   extra_out, (const TW_*)q_w, (const TW_*)k_w, norm_mode, eps, inv_freq, rot_dim, pairing, row_seq, row_pos, \
                   table, max_blocks, (T_*)q_out, (T_*)k_pages, (T_*)v_pages, heads, kv_heads, D, Dv, bias, rot_amp);       \
        return cml_launch_status();                                                                                        \
    }
#define QP_CASE(T_, TW_, D_, DW_)                                                                                          \
    if (dtype == D_ && w_dtype == DW_) {                                                                                   \
        if (few) QP_LAUNCH(T_, TW_, 1024) else QP_LAUNCH(T_, TW_, 256)                                                     \
    }
    QP_CASE(float, float, CML_DTYPE_F32, CML_DTYPE_F32)
    QP_CASE(bf16, bf16, CML_DTYPE_BF16, CML_DTYPE_BF16)
    QP_CASE(bf16, float, CML_DTYPE_BF16, CML_DTYPE_F32)
    QP_CASE(float, bf16, CML_DTYPE_F32, CML_DTYPE_BF16)
#undef QP_CASE
#undef QP_LAUNCH
    return CML_ERR_BAD_DTYPE;
}

// q [rows, heads x D]; out [rows, heads x Dv] = softmax(...) V, times sigmoid(gate) where
// gate (float [rows, ldg], at column gate_col) is given. window <= 0: all keys. r1, r2 float
// [heads] or null (no penalty).
//
// A block of NW warps owns one (row, head). The visible keys, oldest first, are dealt to the
// warps in runs of whole rounds of 32 (how many depends on the row's position and the window
// alone, not on how the prompt was cut); in a round a lane takes one key for the score (the key
// row read in 16-byte pieces where its size allows) and then columns of the values; each warp
// keeps an online softmax of its run, and the runs are merged in warp order at the end.
// Dynamic shared memory: the query (D floats), then per warp its maximum, its sum and Dv sums.
#define AW_MAX_VREGS 16       // value columns per lane at most: Dv <= 512

template <typename T> struct Piece;                 // 16 bytes of a key row as floats
template <> struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ uint4 raw(const float* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ void load(const float* p, float* f) { unpack(raw(p), f); }
};
template <> struct Piece<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ uint4 raw(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
    static __device__ __forceinline__ void load(const bf16* p, float* f) { unpack(raw(p), f); }
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// With MAPS == 2 (differential attention) a head has two score maps: q and the key rows hold the maps' D channels side
// by side, each map is a softmax of its own over the same keys' values, and the head's output is
//   o = a1 - lambda * a2,   then   o / sqrt(mean(o^2) + norm_eps) * out_scale   over the head's Dv channels.
// softcap > 0: score <- softcap * tanh(score / softcap) before the penalty.
struct AwExtra {
    float softcap;          // 0: none
    float lambda;           // MAPS == 2: the factor of the second map
    float norm_eps;         // MAPS == 2: eps of the norm of the difference
    float out_scale;        // MAPS == 2: what the normed difference is multiplied by
};

template <typename T, int NV, int MAPS>    // NV: value columns per lane, Dv <= 32 * NV
__global__ void __launch_bounds__(512, 1) window_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                        const int* __restrict__ table, int max_blocks, const int* __restrict__ row_seq,
                                        const int* __restrict__ row_pos, const float* __restrict__ r1,
                                        const float* __restrict__ r2, const float* __restrict__ gate, long ldg, int gate_col,
                                        T* __restrict__ out, int heads, int kv_heads, int D, int Dv, int window, float scale,
                                        int chunk, const float* __restrict__ sink, int gate_per_head, const AwExtra ex,
                                        int keep_first, int v_stride) {
    extern __shared__ __align__(16) float aw_sh[];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int r = blockIdx.x / heads, hd = blockIdx.x % heads, g = hd / (heads / kv_heads);
    const int KD = MAPS * D;                                 // channels of a query or key row
    const int PW = MAPS * (Dv + 2);                          // floats a warp leaves for the merge
    float* qs = aw_sh;
    float* part = aw_sh + ((KD + 3) & ~3) + warp * PW;
    // what the first round needs besides the query is asked for before the query is staged
    const int i = row_pos[r];
    int lo = window > 0 ? max(0, i - window + 1) : 0;
    if (chunk > 0) lo = max(lo, i - i % chunk);             // the first position of the row's own block
    // the visible keys in order: the kept first ones that lie before the window, then the window's; key number t of
    // them is position t (t < kept) or lo + t - kept
    const int kept = min(keep_first, lo);
    const int shift = lo - kept;
    const int n_vis = kept + i - lo + 1;
    const int rounds = (n_vis - 1) / 32 + 1;
    const int per_warp = (rounds + nw - 1) / nw;
    const int j_first = 32 * warp * per_warp, j_end = min(n_vis, j_first + 32 * per_warp);
    const int* tb = table + (size_t)row_seq[r] * max_blocks;
    int page_first = -1;
    if (j_first + lane < j_end) page_first = tb[(j_first + lane < kept ? j_first + lane : j_first + lane + shift) / CML_PAGE];
    for (int c = threadIdx.x; c < KD; c += blockDim.x) qs[c] = to_f32(q[((size_t)r * heads + hd) * KD + c]);
    __syncthreads();
    const float p1 = r1 ? r1[hd] : 0.f, p2 = r2 ? r2[hd] : 0.f;
    const bool pieces = (D % Piece<T>::N) == 0;              // a key row (and each map of it) is a whole number of 16-byte pieces
    float m[MAPS], l[MAPS];
    float acc[MAPS][NV];
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        m[mp] = -INFINITY; l[mp] = 0.f;
#pragma unroll
        for (int e = 0; e < NV; ++e) acc[mp][e] = 0.f;
    }
    constexpr int PN = Piece<T>::N;
    constexpr int KB = NV * MAPS >= 16 ? 4 : (NV * MAPS >= 8 ? 8 : 16);   // keys whose values are in flight together
    for (int j0 = j_first; j0 < j_end; j0 += 32) {
        const int jv = j0 + lane;                            // its number among the visible keys
        const int j = jv < kept ? jv : jv + shift;           // its position
        float sc[MAPS];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) sc[mp] = -INFINITY;
        int page = -1;
        if (jv < j_end) {
            page = j0 == j_first ? page_first : tb[j / CML_PAGE];
            if (page >= 0) {
#pragma unroll
                for (int mp = 0; mp < MAPS; ++mp) {
                    const T* kr = k_pages + (((size_t)page * kv_heads + g) * CML_PAGE + j % CML_PAGE) * KD + mp * D;
                    const float* qm = qs + mp * D;
                    float dot = 0.f;
                    if (pieces) {
                        // sixteen 16-byte pieces of the key row in flight (a whole row of 128 bfloat16), then their
                        // products; what is left in fours and singly. The sum runs over the channels in order either way.
                        int c = 0;
                        for (; c + 16 * PN <= D; c += 16 * PN) {
                            uint4 raw[16];
#pragma unroll
                            for (int u = 0; u < 16; ++u) raw[u] = Piece<T>::raw(kr + c + u * PN);
#pragma unroll
                            for (int u = 0; u < 16; ++u) {
                                float kf[PN];
                                Piece<T>::unpack(raw[u], kf);
#pragma unroll
                                for (int x = 0; x < PN; ++x) dot = fmaf(qm[c + u * PN + x], kf[x], dot);
                            }
                        }
                        for (; c + 4 * PN <= D; c += 4 * PN) {
                            uint4 raw[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) raw[u] = Piece<T>::raw(kr + c + u * PN);
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                float kf[PN];
                                Piece<T>::unpack(raw[u], kf);
#pragma unroll
                                for (int x = 0; x < PN; ++x) dot = fmaf(qm[c + u * PN + x], kf[x], dot);
                            }
                        }
                        for (; c < D; c += PN) {
                            float kf[PN];
                            Piece<T>::load(kr + c, kf);
#pragma unroll
                            for (int x = 0; x < PN; ++x) dot = fmaf(qm[c + x], kf[x], dot);
                        }
                    } else {
                        for (int c = 0; c < D; ++c) dot = fmaf(qm[c], to_f32(kr[c]), dot);
                    }
                    float v = dot * scale;
                    if (ex.softcap > 0.f) v = ex.softcap * tanhf(v / ex.softcap);
                    if (r1) v -= p1 * log1pf(p2 * (float)(i - j));
                    sc[mp] = v;
                }
            }
        }
        float p[MAPS];
#pragma unroll
        for (int mp = 0; mp < MAPS; ++mp) {
            const float m_new = fmaxf(m[mp], warp_max(sc[mp]));
            p[mp] = sc[mp] == -INFINITY ? 0.f : expf(sc[mp] - m_new);
            const float fix = m[mp] == -INFINITY ? 0.f : expf(m[mp] - m_new);
            l[mp] = l[mp] * fix + warp_sum(p[mp]);
            m[mp] = m_new;
#pragma unroll
            for (int e = 0; e < NV; ++e) acc[mp][e] *= fix;
        }
        const int nk = min(32, j_end - j0);
        // KB keys at a time: their weights and pages by shuffles first, then all their value loads (each
        // unconditional, of a valid row: a key that does not count has weight zero), then the sums in key order
        for (int t0 = 0; t0 < nk; t0 += KB) {
            float pt[MAPS][KB];
            const T* vr[KB];
#pragma unroll
            for (int u = 0; u < KB; ++u) {
                const int t = min(t0 + u, nk - 1);
                const int pg = __shfl_sync(0xffffffffu, page, t);
#pragma unroll
                for (int mp = 0; mp < MAPS; ++mp) {
                    const float pp = __shfl_sync(0xffffffffu, p[mp], t);
                    pt[mp][u] = (t0 + u < nk && pg >= 0) ? pp : 0.f;
                }
                const int jt = j0 + t < kept ? j0 + t : j0 + t + shift;
                vr[u] = v_pages + (((size_t)max(pg, 0) * kv_heads + g) * CML_PAGE + jt % CML_PAGE) * v_stride;
            }
            float vv[KB][NV];
#pragma unroll
            for (int u = 0; u < KB; ++u)
#pragma unroll
                for (int e = 0; e < NV; ++e) {
                    const int c = lane + 32 * e;
                    vv[u][e] = to_f32(vr[u][c < Dv ? c : 0]);
                }
#pragma unroll
            for (int mp = 0; mp < MAPS; ++mp)
#pragma unroll
                for (int u = 0; u < KB; ++u)
#pragma unroll
                    for (int e = 0; e < NV; ++e) acc[mp][e] = fmaf(pt[mp][u], vv[u][e], acc[mp][e]);
        }
    }
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        if (lane == 0) { part[mp * (Dv + 2)] = m[mp]; part[mp * (Dv + 2) + 1] = l[mp]; }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int c = lane + 32 * e;
            if (c < Dv) part[mp * (Dv + 2) + 2 + c] = acc[mp][e];
        }
    }
    __syncthreads();
    // the runs merged in warp order (warp 0 always has the oldest visible key, so the maximum is finite)
    const float* parts = aw_sh + ((KD + 3) & ~3);
    float top[MAPS], inv[MAPS];
    const float snk = sink ? sink[hd] : -INFINITY;              // one more term of the denominator, without a value
#pragma unroll
    for (int mp = 0; mp < MAPS; ++mp) {
        float tp = -INFINITY;
        for (int w = 0; w < nw; ++w) tp = fmaxf(tp, parts[w * PW + mp * (Dv + 2)]);
        tp = fmaxf(tp, snk);
        float total = 0.f;
        for (int w = 0; w < nw; ++w) {
            const float mw = parts[w * PW + mp * (Dv + 2)];
            if (mw != -INFINITY) total += parts[w * PW + mp * (Dv + 2) + 1] * expf(mw - tp);
        }
        if (sink) total += expf(snk - tp);
        top[mp] = tp;
        inv[mp] = 1.0f / total;
    }
    T* o = out + ((size_t)r * heads + hd) * Dv;
    const float* gt = gate ? gate + (size_t)r * ldg + gate_col + (gate_per_head ? hd : hd * Dv) : nullptr;
    const int gstep = gate_per_head ? 0 : 1;
    auto merged = [&](int mp, int c) -> float {
        float sum = 0.f;
        for (int w = 0; w < nw; ++w) {
            const float mw = parts[w * PW + mp * (Dv + 2)];
            if (mw != -INFINITY) sum += parts[w * PW + mp * (Dv + 2) + 2 + c] * expf(mw - top[mp]);
        }
        return sum * inv[mp];
    };
    if (MAPS == 1) {
        for (int c = threadIdx.x; c < Dv; c += blockDim.x)
            o[c] = from_f32<T>(merged(0, c) * (gt ? sigmoid_w(gt[c * gstep]) : 1.0f));
        return;
    }
    // the difference of the two maps, normed over the head's channels: the differences stand behind the warps' parts
    float* diff = aw_sh + ((KD + 3) & ~3) + nw * PW;
    float* red = diff + ((Dv + 3) & ~3);
    float ss = 0.f;
    for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
        const float d = merged(0, c) - ex.lambda * merged(MAPS - 1, c);
        diff[c] = d;
        ss = fmaf(d, d, ss);
    }
    const float rs = ex.out_scale / sqrtf(block_sum(ss, red) / (float)Dv + ex.norm_eps);
    for (int c = threadIdx.x; c < Dv; c += blockDim.x)               // each thread reads back what it wrote itself
        o[c] = from_f32<T>(diff[c] * rs * (gt ? sigmoid_w(gt[c * gstep]) : 1.0f));
}

extern "C" int cml_window_attention(const void* q, const void* k_pages, const void* v_pages, int dtype, const int* table,
                                    int max_blocks, const int* row_seq, const int* row_pos, const float* r1, const float* r2,
                                    const float* gate, long ldg, int gate_col, void* out, int rows, int heads, int kv_heads,
                                    int D, int Dv, int window, float scale, int chunk, const float* sink, int gate_per_head,
                                    int maps, float softcap, float lambda, float norm_eps, float out_scale, int keep_first,
                                    int v_stride, void* stream) {
    if (rows <= 0) return 0;
    if (Dv > 32 * AW_MAX_VREGS || D < 1 || heads % kv_heads || (maps != 1 && maps != 2)) return CML_ERR_BAD_SIZE;
    if (keep_first < 0 || v_stride < Dv || (maps == 2 && Dv > 256)) return CML_ERR_BAD_SIZE;
    // warps per (row, head): one per round of 32 keys of the window, at most 16 (8 without a window); fixed by
    // the window alone, so a row's sums do not depend on the step it came in
    // (or by the block of positions, whichever lets a query see fewer keys)
    if (window <= 0 || chunk > 0) keep_first = 0;               // kept keys go with a window alone
    int span = window > 0 ? window + keep_first : 0;
    if (chunk > 0 && (span == 0 || chunk < span)) span = chunk;
    const int nw = span > 0 ? ((span + 31) / 32 < 16 ? (span + 31) / 32 : 16) : 8;
    dim3 grid((unsigned)((long)rows * heads));
    const size_t smem = (size_t)(((maps * D + 3) & ~3) + nw * maps * (Dv + 2) + (maps > 1 ? ((Dv + 3) & ~3) + 32 : 0)) * sizeof(float);
    if (smem > 48 * 1024 || (long)rows * heads > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const AwExtra ex = {softcap, lambda, norm_eps, out_scale};
#define AW_CASE(T_, NV_, MP_)                                                                                               \
    launch_pdl(window_attention_kernel<T_, NV_, MP_>, grid, dim3(32 * nw), smem, s, (const T_*)q, (const T_*)k_pages, (const T_*)v_pages, \
               table, max_blocks, row_seq, row_pos, r1, r2, gate, ldg, gate_col, (T_*)out, heads, kv_heads, D, Dv, window, scale, \
               chunk, sink, gate_per_head, ex, keep_first, v_stride)
#define AW_SIZES(T_)                                                                                                        \
    if (maps == 2) { if (Dv <= 32) AW_CASE(T_, 1, 2); else if (Dv <= 64) AW_CASE(T_, 2, 2); else if (Dv <= 128) AW_CASE(T_, 4, 2); else AW_CASE(T_, 8, 2); } \
    else if (Dv <= 32) AW_CASE(T_, 1, 1); else if (Dv <= 64) AW_CASE(T_, 2, 1); else if (Dv <= 128) AW_CASE(T_, 4, 1); \
    else if (Dv <= 256) AW_CASE(T_, 8, 1); else AW_CASE(T_, 16, 1)
    if (dtype == CML_DTYPE_F32) { AW_SIZES(float); }
    else if (dtype == CML_DTYPE_BF16) { AW_SIZES(bf16); }
    else return CML_ERR_BAD_DTYPE;
#undef AW_SIZES
#undef AW_CASE
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// The combination of two score maps that ran as attentions of their own (the tensor-core prompt kernel writes them as
// float rows [head, map, Dv]): per (row, head) o = a1 - lambda a2, then o / sqrt(mean(o^2) + eps) * out_scale over the
// head's Dv channels, written in the compute type. A warp owns one (row, head) and keeps its differences in registers.
template <typename T>
__global__ void maps_difference_kernel(const float* __restrict__ maps_out, long ld, T* __restrict__ out, long ldo, long pairs,
                                       int heads, int Dv, float lambda, float eps, float out_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= pairs) return;
    const long r = warp / heads;
    const int h = (int)(warp % heads);
    const float* a1 = maps_out + r * ld + (size_t)h * 2 * Dv;
    const float* a2 = a1 + Dv;
    float d[AW_MAX_VREGS];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < AW_MAX_VREGS; ++j) {
        const int c = lane + 32 * j;
        d[j] = c < Dv ? a1[c] - lambda * a2[c] : 0.f;
        ss = fmaf(d[j], d[j], ss);
    }
    const float rs = out_scale / sqrtf(warp_sum(ss) / (float)Dv + eps);
    T* o = out + r * ldo + (size_t)h * Dv;
#pragma unroll
    for (int j = 0; j < AW_MAX_VREGS; ++j) {
        const int c = lane + 32 * j;
        if (c < Dv) o[c] = from_f32<T>(d[j] * rs);
    }
}

extern "C" int cml_maps_difference(const void* maps_out, long ld, void* out, long ldo, int dtype, long rows, int heads, int Dv,
                                   float lambda, float eps, float out_scale, void* stream) {
    if (rows <= 0) return 0;
    if (heads < 1 || Dv < 1 || Dv > 32 * AW_MAX_VREGS) return CML_ERR_BAD_SIZE;
    const long pairs = rows * heads;
    const long blocks = (pairs + 7) / 8;
    if (blocks > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CML_DTYPE_BF16)
        launch_pdl(maps_difference_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, s, (const float*)maps_out, ld, (bf16*)out,
                   ldo, pairs, heads, Dv, lambda, eps, out_scale);
    else if (dtype == CML_DTYPE_F32)
        launch_pdl(maps_difference_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, (const float*)maps_out, ld, (float*)out,
                   ldo, pairs, heads, Dv, lambda, eps, out_scale);
    else return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
