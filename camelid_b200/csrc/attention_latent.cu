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

// 16-byte asynchronous copies into shared memory, matrix fragments out of it, and the bfloat16 tensor-core instruction
// (m16n8k16, float accumulation) that the prompt kernel and the product per head use.
__device__ __forceinline__ void la_cp16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void la_ldmatrix4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void la_ldmatrix4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// (the same two by a 32-bit shared-memory address, for loops that step through a tile with plain adds)
__device__ __forceinline__ uint32_t la_smem32(const void* smem) { return (uint32_t)__cvta_generic_to_shared(smem); }
__device__ __forceinline__ void la_ldsm4(uint32_t (&r)[4], uint32_t s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void la_ldsm4_trans(uint32_t (&r)[4], uint32_t s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void la_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t la_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}


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

// The same product for a step of few rows (single tokens): a warp owns one output n of one head, reads its weight row
// w[h, n, :] once in 16-byte pieces and multiplies it with every row's x (staged in shared memory as floats); the sums
// over K are reduced over the lanes in a fixed order. Rows <= HPF_ROWS.
#define HPF_ROWS 16
template <typename T>
__global__ void __launch_bounds__(256) head_product_few_kernel(const T* __restrict__ x, long ldx, int xs, const T* __restrict__ w,
                                                               T* __restrict__ out, long ldo, int os, int rows, int N, int K) {
    extern __shared__ __align__(16) float hx[];                    // [rows][K]
    pdl_wait();
    pdl_launch_dependents();
    const int hd = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < rows * K; i += 256) {
        const int r = i / K, k = i - r * K;
        hx[i] = to_f32(x[(size_t)r * ldx + (size_t)hd * xs + k]);
    }
    __syncthreads();
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const T* wr = w + ((size_t)hd * N + n) * K;
    float acc[HPF_ROWS];
#pragma unroll
    for (int r = 0; r < HPF_ROWS; ++r) acc[r] = 0.f;
    constexpr int PIECE = 16 / sizeof(T);
    if ((K % PIECE) == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int k = lane * PIECE; k < K; k += 32 * PIECE) {
            union { uint4 raw; T e[PIECE]; } v;
            v.raw = *reinterpret_cast<const uint4*>(wr + k);
#pragma unroll
            for (int r = 0; r < HPF_ROWS; ++r) {
                if (r < rows) {
#pragma unroll
                    for (int e = 0; e < PIECE; ++e) acc[r] = fmaf(hx[r * K + k + e], to_f32(v.e[e]), acc[r]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32(wr[k]);
#pragma unroll
            for (int r = 0; r < HPF_ROWS; ++r)
                if (r < rows) acc[r] = fmaf(hx[r * K + k], wv, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < HPF_ROWS; ++r) {
        if (r < rows) {
            const float v = warp_sum(acc[r]);
            if (lane == 0) out[(size_t)r * ldo + (size_t)hd * os + n] = from_f32<T>(v);
        }
    }
}

// The same product in bfloat16 on the tensor cores (mma.sync m16n8k16) for steps of many rows: a block of four warps owns
// 64 rows x 64 outputs of one head, a warp 16 of the rows; K passes through shared memory 64 channels at a time (rows
// 16 bytes longer than the data against bank conflicts). Needs K mod 16 = 0 and 16-byte aligned rows of x and w.
#define HPT_TILE 64
__global__ void __launch_bounds__(128) head_product_mma_kernel(const bf16* __restrict__ x, long ldx, int xs, const bf16* __restrict__ w,
                                                               bf16* __restrict__ out, long ldo, int os, int rows, int N, int K) {
    constexpr int PITCH = HPT_TILE * 2 + 16;
    __shared__ __align__(16) unsigned char sx[HPT_TILE * PITCH];
    __shared__ __align__(16) unsigned char sw[HPT_TILE * PITCH];
    pdl_wait();
    pdl_launch_dependents();
    const int hd = blockIdx.z, r0 = blockIdx.y * HPT_TILE, n0 = blockIdx.x * HPT_TILE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* wh = w + (size_t)hd * N * K;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HPT_TILE) {
        const int kc = min(HPT_TILE, K - k0);                      // a multiple of 16
        for (int i = threadIdx.x; i < HPT_TILE * 8; i += 128) {
            const int r = i >> 3, c = i & 7;
            unsigned char* dx = sx + r * PITCH + c * 16;
            unsigned char* dw = sw + r * PITCH + c * 16;
            if (r0 + r < rows && c * 8 < kc) la_cp16(dx, x + (size_t)(r0 + r) * ldx + (size_t)hd * xs + k0 + c * 8);
            else *reinterpret_cast<uint4*>(dx) = make_uint4(0u, 0u, 0u, 0u);
            if (n0 + r < N && c * 8 < kc) la_cp16(dw, wh + (size_t)(n0 + r) * K + k0 + c * 8);
            else *reinterpret_cast<uint4*>(dw) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        for (int kk = 0; kk < kc; kk += 16) {
            uint32_t a[4];
            la_ldmatrix4(a, sx + (warp * 16 + (lane & 15)) * PITCH + (kk + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int nj = 0; nj < 4; ++nj) {
                uint32_t b[4];
                la_ldmatrix4(b, sw + (nj * 16 + (lane & 7) + (lane >> 4) * 8) * PITCH + (kk + ((lane >> 3) & 1) * 8) * 2);
                la_mma(acc[2 * nj], a, b[0], b[1]);
                la_mma(acc[2 * nj + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = r0 + warp * 16 + (lane >> 2) + 8 * h;
        if (r >= rows) continue;
        bf16* orow = out + (size_t)r * ldo + (size_t)hd * os;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const int c = n0 + n * 8 + 2 * (lane & 3);
            if (c < N) orow[c] = __float2bfloat16_rn(acc[n][2 * h]);
            if (c + 1 < N) orow[c + 1] = __float2bfloat16_rn(acc[n][2 * h + 1]);
        }
    }
}

extern "C" int cml_head_product(const void* x, long ldx, int xs, const void* w, void* out, long ldo, int os, int dtype, int rows,
                                int heads, int N, int K, void* stream) {
    if (rows <= 0 || heads <= 0 || N <= 0) return 0;
    if (K < 1 || heads > 65535 || (rows + HP_ROWS - 1) / HP_ROWS > 65535) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t few_smem = (size_t)rows * K * sizeof(float);
    if (rows <= HPF_ROWS && few_smem <= 48 * 1024) {
        dim3 grid_few((unsigned)((N + 7) / 8), (unsigned)heads);
        if (dtype == CML_DTYPE_F32)
            launch_pdl(head_product_few_kernel<float>, grid_few, dim3(256), few_smem, s, (const float*)x, ldx, xs, (const float*)w,
                       (float*)out, ldo, os, rows, N, K);
        else if (dtype == CML_DTYPE_BF16)
            launch_pdl(head_product_few_kernel<bf16>, grid_few, dim3(256), few_smem, s, (const bf16*)x, ldx, xs, (const bf16*)w,
                       (bf16*)out, ldo, os, rows, N, K);
        else
            return CML_ERR_BAD_DTYPE;
        return cml_launch_status();
    }
    if (dtype == CML_DTYPE_BF16 && (K & 15) == 0 && (ldx & 7) == 0 && (xs & 7) == 0 && ((((uintptr_t)x) | ((uintptr_t)w)) & 15) == 0 &&
        (rows + HPT_TILE - 1) / HPT_TILE <= 65535) {
        dim3 grid_mma((unsigned)((N + HPT_TILE - 1) / HPT_TILE), (unsigned)((rows + HPT_TILE - 1) / HPT_TILE), (unsigned)heads);
        launch_pdl(head_product_mma_kernel, grid_mma, dim3(128), 0, s, (const bf16*)x, ldx, xs, (const bf16*)w, (bf16*)out, ldo, os,
                   rows, N, K);
        return cml_launch_status();
    }
    dim3 grid((unsigned)((N + HP_COLS - 1) / HP_COLS), (unsigned)((rows + HP_ROWS - 1) / HP_ROWS), (unsigned)heads);
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

// ------------------------------------------------------------------------------------
// Prompts in bfloat16 on the tensor cores (mma.sync m16n8k16, float accumulation). All query heads share the one row
// [c_j, t_j] per position, so a block takes 64 (token, head) query rows of one sequence against pages of 64 keys: the
// page is fetched once (cp.async, the next one while this one is worked on) and serves as keys (all C + R channels) and
// as values (its first C channels). Eight warps: warps w and w + 4 share rows 16 (w mod 4) .. + 15; each computes the
// scores of half of the page's keys and owns half of the value channels. Through shared memory (and a barrier of
// their own, twice a page) the two exchange their rows' maxima, so that both use the same reference, and their halves
// of the weights, packed as the second product's operand. Scores, running maximum and sum are float; the weights
// enter the second product as bfloat16. The sink's term joins the denominator at the end; a head's gate (one number) scales its row. Single
// tokens run here too: a tile is then one token's heads, and a long context is dealt to several blocks by pages.
//
// Rows of a tile: local row i is token i / HB of the tile and head chunk * HB + i mod HB, with HB = min(heads, 64) heads a
// tile and 64 / HB tokens (one where there are more than 64 heads). Shared memory rows are 16 bytes longer than the
// data, so that eight rows of a ldmatrix fall into different banks. Needs C mod 32 = 0 and R mod 16 = 0.
#define LA_ROWS 64
#define LA_KEYS 64

struct LatentPromptParams {
    const bf16* q;          // [rows, heads x (C + R)]
    const bf16* k_pages;    // [pages, 1, 64, C + R]
    bf16* out;              // [rows, heads x C]
    const int* table; int max_blocks;
    const int* tile_seq; const int* tile_q0; int n_tiles; int tokens_per_tile;
    const int* seq_row0; const int* seq_start; const int* seq_new;
    const float* sink;      // [heads] or null
    const float* gate; long gate_ld; int gate_col;      // float [rows, gate_ld] or null: one logit per head
    int heads, C, R;
    float scale;
    // single tokens over long contexts: a sequence's pages are dealt to gridDim.y blocks, `tiles_per_split` pages each; every
    // block leaves its rows' maximum (scaled), sum and unnormalised sums as floats in `partial`
    // [split, row, head, 2 + C], and a second kernel merges them (and adds the sink's term and the gate)
    float* partial; int tiles_per_split; long rows_total;
};

template <int NG>           // groups of 16 value channels a warp owns at most: C / 2 <= 16 NG
__global__ void __launch_bounds__(256, 1) latent_prompt_kernel(const LatentPromptParams p) {
    extern __shared__ __align__(16) unsigned char la_smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int D = p.C + p.R;
    const int pitch = D * 2 + 16;                                  // bytes of a shared-memory row
    unsigned char* sQ = la_smem;
    unsigned char* sK = la_smem + (size_t)LA_ROWS * pitch;         // two buffers of LA_KEYS rows
    // behind them: what a warp hands its partner, [warp][16-key step][register][lane]; the rows' maxima and sums go
    // through the 16 spare bytes at the end of the query rows
    uint32_t* sX = reinterpret_cast<uint32_t*>(la_smem + (size_t)(LA_ROWS + 2 * LA_KEYS) * pitch);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int HB = min(p.heads, LA_ROWS), chunks = (p.heads + HB - 1) / HB;
    // blocks in the order of blockIdx.x: the tiles that see the most keys first
    const int tile = p.n_tiles - 1 - (int)(blockIdx.x / chunks), chunk = (int)(blockIdx.x % chunks);
    const int seq = p.tile_seq[tile], q0 = p.tile_q0[tile];
    const int start = p.seq_start[seq], n_new = p.seq_new[seq], row0 = p.seq_row0[seq];
    const int tokens = min(p.tokens_per_tile, n_new - q0);
    const int all_key_tiles = (start + q0 + tokens + LA_KEYS - 1) / LA_KEYS;
    const int t_begin = p.partial ? min((int)blockIdx.y * p.tiles_per_split, all_key_tiles) : 0;
    const int n_key_tiles = p.partial ? min(t_begin + p.tiles_per_split, all_key_tiles) : all_key_tiles;
    const int* tb = p.table + (size_t)seq * p.max_blocks;
    const int chunks16 = D / 8;                                    // 16-byte pieces of a row
    auto fetch_keys = [&](int t, int buf) {
        const int page = tb[t];
        const bf16* src = p.k_pages + (size_t)max(page, 0) * CML_PAGE * D;
        unsigned char* dst = sK + (size_t)buf * LA_KEYS * pitch;
        // a warp takes every eighth row, a lane every 32nd piece of it (no division by a size known only at run time)
        for (int r = threadIdx.x >> 5; r < LA_KEYS; r += 8)
            for (int c = threadIdx.x & 31; c < chunks16; c += 32)
                la_cp16(dst + (size_t)r * pitch + c * 16, src + (size_t)r * D + c * 8);
    };
    // the queries: rows that stand for nothing hold zeros
    for (int r = threadIdx.x >> 5; r < LA_ROWS; r += 8) {
        const int tok = r / HB, hd = chunk * HB + r % HB;
        const bool there = tok < tokens && hd < p.heads;
        const bf16* src = p.q + ((size_t)(row0 + q0 + (there ? tok : 0)) * p.heads + (there ? hd : 0)) * D;
        for (int c = threadIdx.x & 31; c < chunks16; c += 32) {
            unsigned char* dst = sQ + (size_t)r * pitch + c * 16;
            if (there) la_cp16(dst, src + c * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    if (t_begin < n_key_tiles) fetch_keys(t_begin, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    const int wrow = (warp & 3) * 16;                              // the warp's rows of the tile
    const int half = warp >> 2;                                    // its half of the page's keys and of the value channels
    const int kb = half * (LA_KEYS / 2);
    auto pair_barrier = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory"); };
    // a row's number handed to the partner: slot `half` of the row's spare bytes; returns the partner's
    auto swap_rows = [&](const float (&mine)[2], float (&theirs)[2]) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
            if ((lane & 3) == 0)
                *reinterpret_cast<float*>(sQ + (size_t)(wrow + (lane >> 2) + 8 * h) * pitch + D * 2 + half * 4) = mine[h];
        pair_barrier();
#pragma unroll
        for (int h = 0; h < 2; ++h)
            theirs[h] = *reinterpret_cast<const float*>(sQ + (size_t)(wrow + (lane >> 2) + 8 * h) * pitch + D * 2 + (half ^ 1) * 4);
    };
    const int n_groups = p.C / 32;                                 // groups of 16 channels in a half
    const int ch0 = half * (p.C / 2);
    // the two rows a lane holds pieces of: wrow + lane / 4 and that + 8
    int pos[2];
    bool valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wrow + (lane >> 2) + 8 * h;
        const int tok = r / HB, hd = chunk * HB + r % HB;
        valid[h] = tok < tokens && hd < p.heads;
        pos[h] = valid[h] ? start + q0 + tok : 0x7fffffff;         // rows that stand for nothing see everything: no empty softmax
    }
    float o[NG][2][4];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[g][j][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float sl2 = p.scale * 1.4426950408889634f;

    for (int t = t_begin; t < n_key_tiles; ++t) {
        if (t + 1 < n_key_tiles) fetch_keys(t + 1, (t + 1 - t_begin) & 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");       // everything but the newest group: this tile (and Q) is here
        __syncthreads();
        const unsigned char* kt = sK + (size_t)((t - t_begin) & 1) * LA_KEYS * pitch;
        float s[4][4];                                             // this warp's 32 keys of the page
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
        {   // 16 channels a step; the fragments of the next step are asked for before this step's products are issued
            const uint32_t qa = la_smem32(sQ) + (uint32_t)((wrow + (lane & 15)) * pitch + (lane >> 4) * 16);
            const uint32_t ka = la_smem32(kt) + (uint32_t)((kb + (lane & 7) + (lane >> 4) * 8) * pitch + ((lane >> 3) & 1) * 16);
            const uint32_t kstep = (uint32_t)(16 * pitch);         // the second pair of key tiles
            const int nk = D / 16;
            uint32_t a0[4], b00[4], b01[4], a1[4], b10[4], b11[4];
            la_ldsm4(a0, qa); la_ldsm4(b00, ka); la_ldsm4(b01, ka + kstep);
            int ks = 0;
            for (; ks + 2 <= nk; ks += 2) {
                const uint32_t o1 = (uint32_t)(ks + 1) * 32u;
                la_ldsm4(a1, qa + o1); la_ldsm4(b10, ka + o1); la_ldsm4(b11, ka + kstep + o1);
                la_mma(s[0], a0, b00[0], b00[1]); la_mma(s[1], a0, b00[2], b00[3]);
                la_mma(s[2], a0, b01[0], b01[1]); la_mma(s[3], a0, b01[2], b01[3]);
                if (ks + 2 < nk) {
                    const uint32_t o2 = (uint32_t)(ks + 2) * 32u;
                    la_ldsm4(a0, qa + o2); la_ldsm4(b00, ka + o2); la_ldsm4(b01, ka + kstep + o2);
                }
                la_mma(s[0], a1, b10[0], b10[1]); la_mma(s[1], a1, b10[2], b10[3]);
                la_mma(s[2], a1, b11[0], b11[1]); la_mma(s[3], a1, b11[2], b11[3]);
            }
            if (ks < nk) {                                         // an odd number of steps: the last one is loaded already
                la_mma(s[0], a0, b00[0], b00[1]); la_mma(s[1], a0, b00[2], b00[3]);
                la_mma(s[2], a0, b01[0], b01[1]); la_mma(s[3], a0, b01[2], b01[3]);
            }
        }
        // mask and maximum per row: a row's 32 scores lie in the four lanes of a quad, the other 32 with the partner
        const int key0 = t * LA_KEYS + kb + 2 * (lane & 3);
        float mx[2] = {-INFINITY, -INFINITY};
        const bool page_whole = (t + 1) * LA_KEYS - 1 <= start + q0;      // every row of the tile sees all of this page
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + 8 * n + (e & 1), h = e >> 1;
                if (!page_whole && key > pos[h]) s[n][e] = -INFINITY;
                mx[h] = fmaxf(mx[h], s[n][e]);
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        }
        float mx_other[2];
        swap_rows(mx, mx_other);
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], mx_other[h]);
            const float m_new = fmaxf(m[h], mx[h]);                // finite from a sequence's first page on: key 0 is visible to every row
            corr[h] = m[h] == -INFINITY ? 0.f : exp2f((m[h] - m_new) * sl2);
            m[h] = m_new;
        }
        uint32_t pa[4][4], mine[2][4], theirs[2][4];               // the weights as the first operand of the second product
        float sum[2] = {0.f, 0.f};
        // (a row that has seen no key yet, in a block that starts at a later page, keeps weights of zero)
        const float mref[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            float e4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                e4[e] = exp2f((s[n][e] - mref[e >> 1]) * sl2);
                sum[e >> 1] += e4[e];
            }
            mine[n >> 1][(n & 1) * 2] = la_pack(e4[0], e4[1]);
            mine[n >> 1][(n & 1) * 2 + 1] = la_pack(e4[2], e4[3]);
        }
        // this warp's two steps of 16 keys to the partner, the partner's two from it
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sX[((warp * 2 + i) * 4 + e) * 32 + lane] = mine[i][e];
        pair_barrier();
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) theirs[i][e] = sX[(((warp ^ 4) * 2 + i) * 4 + e) * 32 + lane];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)                             // in the order of the keys: the lower half's steps first
#pragma unroll
            for (int e = 0; e < 4; ++e) pa[kk][e] = ((kk >> 1) == half) ? mine[kk & 1][e] : theirs[kk & 1][e];
#pragma unroll
        for (int h = 0; h < 2; ++h) l[h] = l[h] * corr[h] + sum[h];
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {      // a maximum moved in one of the warp's rows
#pragma unroll
            for (int g = 0; g < NG; ++g)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    o[g][j][0] *= corr[0]; o[g][j][1] *= corr[0];
                    o[g][j][2] *= corr[1]; o[g][j][3] *= corr[1];
                }
        }
        // weights times values: 16 keys a step, 16 channels a group
        const uint32_t va = la_smem32(kt) + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (ch0 + (lane >> 4) * 8) * 2);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t vb[2][4];                                     // the next group's fragment is asked for before this one's products
            la_ldsm4_trans(vb[0], va + (uint32_t)(kk * 16 * pitch));
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                if (g < n_groups) {
                    if (g + 1 < n_groups) la_ldsm4_trans(vb[(g + 1) & 1], va + (uint32_t)(kk * 16 * pitch + (g + 1) * 32));
                    la_mma(o[g][0], pa[kk], vb[g & 1][0], vb[g & 1][1]);
                    la_mma(o[g][1], pa[kk], vb[g & 1][2], vb[g & 1][3]);
                }
            }
        }
        __syncthreads();                                           // before the next fetch overwrites this buffer
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the rows' sums over their quads and both warps of the pair (in the order of the keys), the sink's term, the gate
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    {
        float l_other[2];
        swap_rows(l, l_other);
#pragma unroll
        for (int h = 0; h < 2; ++h) l[h] = half == 0 ? l[h] + l_other[h] : l_other[h] + l[h];
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!valid[h]) continue;
        const int r = wrow + (lane >> 2) + 8 * h;
        const int tok = r / HB, hd = chunk * HB + r % HB;
        const size_t grow = (size_t)(row0 + q0 + tok);
        if (p.partial != nullptr) {                                // this block's share, for the merge
            float* part = p.partial + (((size_t)blockIdx.y * p.rows_total + grow) * p.heads + hd) * (p.C + 2);
            if (half == 0 && (lane & 3) == 0) { part[0] = m[h] * p.scale; part[1] = l[h]; }
            float* prow = part + 2 + ch0 + 2 * (lane & 3);
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                if (g < n_groups) {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        *reinterpret_cast<float2*>(prow + g * 16 + j * 8) = make_float2(o[g][j][2 * h], o[g][j][2 * h + 1]);
                }
            }
            continue;
        }
        float top = m[h] * p.scale, total = l[h];                  // the scores' maximum, scaled, and the sum against it
        if (p.sink != nullptr) {
            const float snk = p.sink[hd];
            const float top2 = fmaxf(top, snk);
            const float back = expf(top - top2);
            total = total * back + expf(snk - top2);
            total /= back;                                         // the rows in `o` stand against `top`
        }
        float f = 1.0f / total;
        if (p.gate != nullptr) f *= 1.0f / (1.0f + expf(-p.gate[grow * p.gate_ld + p.gate_col + hd]));
        bf16* orow = p.out + (grow * p.heads + hd) * p.C + ch0 + 2 * (lane & 3);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            if (g < n_groups) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t v = la_pack(o[g][j][2 * h] * f, o[g][j][2 * h + 1] * f);
                    *reinterpret_cast<uint32_t*>(orow + g * 16 + j * 8) = v;
                }
            }
        }
    }
}

// The shares of a row's key ranges merged in split order: out[row, head] = sum_s o_s e^(m_s - top) / (sum_s l_s e^(m_s - top)
// + e^(sink - top)) times sigmoid(gate). One block per (row, head).
__global__ void latent_merge_kernel(const float* __restrict__ partial, int n_splits, long rows_total, bf16* __restrict__ out,
                                    const float* __restrict__ sink, const float* __restrict__ gate, long gate_ld, int gate_col,
                                    int heads, int C) {
    pdl_wait();
    pdl_launch_dependents();
    const long r = blockIdx.x / heads;
    const int hd = blockIdx.x % heads;
    const size_t stride = (size_t)rows_total * heads * (C + 2);
    const float* first = partial + ((size_t)r * heads + hd) * (C + 2);
    const float snk = sink ? sink[hd] : -INFINITY;
    float top = snk;
    for (int s = 0; s < n_splits; ++s) top = fmaxf(top, first[s * stride]);
    float total = sink ? expf(snk - top) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = first[s * stride];
        if (ms != -INFINITY) total += first[s * stride + 1] * expf(ms - top);
    }
    float f = 1.0f / total;
    if (gate != nullptr) f *= 1.0f / (1.0f + expf(-gate[r * gate_ld + gate_col + hd]));
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = first[s * stride];
            if (ms != -INFINITY) acc += first[s * stride + 2 + c] * expf(ms - top);
        }
        out[((size_t)r * heads + hd) * C + c] = __float2bfloat16_rn(acc * f);
    }
}

extern "C" int cml_latent_prompt_tokens_per_tile(int heads) { return heads >= LA_ROWS ? 1 : LA_ROWS / heads; }

extern "C" int cml_latent_prompt(const void* q, const void* k_pages, void* out, const int* table, int max_blocks,
                                 const int* tile_seq, const int* tile_q0, int n_tiles, int tokens_per_tile, const int* seq_row0,
                                 const int* seq_start, const int* seq_new, const float* sink, const float* gate, long gate_ld,
                                 int gate_col, int heads, int C, int R, float scale, float* partial, int n_splits,
                                 int tiles_per_split, long rows_total, void* stream) {
    if (n_tiles <= 0) return 0;
    if (partial != nullptr && (n_splits < 1 || n_splits > 65535 || tiles_per_split < 1 || tokens_per_tile != 1)) return CML_ERR_BAD_SIZE;
    if (heads < 1 || C < 32 || (C & 31) || (R & 15) || C > 512 || R < 0) return CML_ERR_BAD_SIZE;
    const int HB = heads < LA_ROWS ? heads : LA_ROWS;
    if (tokens_per_tile < 1 || tokens_per_tile * HB > LA_ROWS) return CML_ERR_BAD_SIZE;
    if ((((uintptr_t)q) | ((uintptr_t)k_pages) | ((uintptr_t)out)) & 15) return CML_ERR_BAD_ALIGN;
    const int chunks = (heads + HB - 1) / HB;
    if ((long)n_tiles * chunks > 0x7fffffffL) return CML_ERR_BAD_SIZE;
    LatentPromptParams p;
    p.q = (const bf16*)q; p.k_pages = (const bf16*)k_pages; p.out = (bf16*)out; p.table = table; p.max_blocks = max_blocks;
    p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.n_tiles = n_tiles; p.tokens_per_tile = tokens_per_tile;
    p.seq_row0 = seq_row0; p.seq_start = seq_start; p.seq_new = seq_new; p.sink = sink; p.gate = gate; p.gate_ld = gate_ld;
    p.gate_col = gate_col; p.heads = heads; p.C = C; p.R = R; p.scale = scale;
    p.partial = partial; p.tiles_per_split = tiles_per_split; p.rows_total = rows_total;
    const size_t smem = (size_t)(LA_ROWS + 2 * LA_KEYS) * ((C + R) * 2 + 16) + 8 * 2 * 4 * 32 * sizeof(uint32_t);
    if (smem > 227 * 1024) return CML_ERR_BAD_SIZE;
    dim3 grid((unsigned)(n_tiles * chunks), partial ? (unsigned)n_splits : 1u);
    cudaStream_t s = (cudaStream_t)stream;
#define LPK_CASE(NG_)                                                                                        \
    {                                                                                                        \
        if (smem > 48 * 1024 && cml_allow_smem<latent_prompt_kernel<NG_>>(smem) != cudaSuccess) return CML_ERR_BAD_SIZE; \
        launch_pdl(latent_prompt_kernel<NG_>, grid, dim3(256), smem, s, p);                                  \
        int rc = cml_launch_status();                                                                        \
        if (rc == 0 && partial != nullptr) {                                                                 \
            launch_pdl(latent_merge_kernel, dim3((unsigned)(rows_total * heads)), dim3(128), 0, s, (const float*)partial, n_splits, \
                       rows_total, (bf16*)out, sink, gate, gate_ld, gate_col, heads, C);                     \
            rc = cml_launch_status();                                                                        \
        }                                                                                                    \
        return rc;                                                                                           \
    }
    if (C <= 128) LPK_CASE(4)
    if (C <= 256) LPK_CASE(8)
    LPK_CASE(16)
#undef LPK_CASE
}
