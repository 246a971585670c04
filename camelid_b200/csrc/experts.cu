// Routed feed-forwards (mixtures of experts): every row picks its `top` experts by float32 router
// logits; the (row, choice) pairs are ordered by expert so that each expert's rows lie together, the
// experts' products run as one grouped launch over those stretches, and the rows' results are added
// back in the order of the choices. Nothing here is read on the host: counts, offsets and the tiles of
// the grouped products live in device memory, so a step with experts replays inside a captured graph.
//
//   route_topk      logits [rows, E] -> ids, weights [rows, top]   (sigmoid of the logit, or softmax over E)
//   expert_rank     for expert e (one block each): the rank of each of its pairs among them, and their count
//   expert_offsets  exclusive sums of the counts and of the counts' tiles of `tile_rows` rows (64 for the product
//                   below, 128 for the grouped product on the tensor cores)
//   expert_gather   xs[offset[e] + rank] = x[row] (* weight): the experts' inputs, ordered by expert
//   expert_gemm     C[pos] = xs[pos] W_e^T per stretch; plain float store, or silu(gate) * up in the compute type
//   expert_combine  out[row] = shared[row] + sum over the row's choices of y[pos] (* weight)
#define CML_HAS_GATE_ACT
#include "common.cuh"

#define EX_TM 64            // rows of a tile of the grouped product
#define EX_TN 64
#define EX_TK 16

// One warp per row. A lane looks after experts lane, lane + 32, ...; a chosen expert is marked in the lane's
// bit mask (so at most 1,024 experts). Ties go to the lower index.
// The logits may come as split sums (n_splits matrices split_stride apart): a warp adds them, in split order, into its
// own stretch of shared memory first.
// The choice may be made on other numbers than the weights: `correction` [E] (may be null) is added to the scores
// for the choice alone, and with n_groups > 1 the experts form n_groups equal groups of neighbours of which only
// the `keep_groups` with the largest choice score of any member stay open (the others' choice scores count as
// minus infinity). The weights are the chosen experts' uncorrected scores times `weight_scale`.
// Shared memory per warp: the scores (E floats), the choice scores (E floats), the groups' best (n_groups floats).
__global__ void route_topk_kernel(const float* __restrict__ logits, long ld, int n_splits, long split_stride, int rows, int E,
                                  int top, int score_mode, int renorm, const float* __restrict__ correction, int n_groups,
                                  int keep_groups, float weight_scale, int* __restrict__ ids, float* __restrict__ wts) {
    extern __shared__ float rt_z[];
    pdl_wait();
    pdl_launch_dependents();
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= rows) return;
    const bool separate = correction != nullptr || n_groups > 1;   // the choice runs on numbers of its own
    const int per_warp = separate ? 2 * E + n_groups : E;
    float* z = rt_z + (threadIdx.x >> 5) * per_warp;
    float* ch = separate ? z + E : z;
    float* gbest = z + 2 * E;
    for (int e = lane; e < E; e += 32) {
        float v = logits[(size_t)r * ld + e];
        for (int s0 = 1; s0 < n_splits; s0 += 8) {              // eight splits' loads in flight, added in split order
            float t[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = logits[(size_t)min(s0 + k, n_splits - 1) * split_stride + (size_t)r * ld + e];
#pragma unroll
            for (int k = 0; k < 8; ++k) v += s0 + k < n_splits ? t[k] : 0.f;
        }
        z[e] = v;
    }
    __syncwarp();
    float zmax = -INFINITY, zsum = 0.f;
    if (score_mode == 1) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(z[e] - zmax);
        zsum = warp_sum(zsum);
    }
    if (separate) {
        // scores in place of the logits, choice scores beside them
        for (int e = lane; e < E; e += 32) {
            const float sc = score_mode == 1 ? expf(z[e] - zmax) / zsum : 1.0f / (1.0f + expf(-z[e]));
            z[e] = sc;
            ch[e] = correction ? sc + correction[e] : sc;
        }
        __syncwarp();
        if (n_groups > 1) {
            const int per = E / n_groups;
            for (int g = lane; g < n_groups; g += 32) {
                float b = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, ch[e]);
                gbest[g] = b;
            }
            __syncwarp();
            // a group stays open if fewer than keep_groups groups come before it (larger best, or equal and lower number)
            for (int e = lane; e < E; e += 32) {
                const int g = e / per;
                const float mine = gbest[g];
                int before = 0;
                for (int o = 0; o < n_groups; ++o) before += (gbest[o] > mine || (gbest[o] == mine && o < g)) ? 1 : 0;
                if (before >= keep_groups) ch[e] = -INFINITY;
            }
            __syncwarp();
        }
    }
    unsigned taken = 0u;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int t = 0, e = lane; e < E; ++t, e += 32) {
            const float v = ch[e];
            if (!((taken >> t) & 1u) && (v > best || at == 0x7fffffff)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) at = 0;                           // fewer experts than choices: never for a valid model
        if ((at & 31) == lane) taken |= 1u << (at >> 5);
        float w;
        if (separate) w = z[at];
        else w = score_mode == 1 ? expf(best - zmax) / zsum : 1.0f / (1.0f + expf(-best));
        w *= weight_scale;
        total += w;
        if (lane == 0) { ids[(size_t)r * top + k] = at; wts[(size_t)r * top + k] = w; }
    }
    if (renorm) {                                               // the chosen weights divided by their sum
        __syncwarp();
        for (int k = lane; k < top; k += 32) wts[(size_t)r * top + k] *= weight_scale / total;
    }
}

extern "C" int cml_route_topk(const float* logits, long ld, int n_splits, long split_stride, int rows, int E, int top,
                              int score_mode, int renorm, const float* correction, int n_groups, int keep_groups,
                              float weight_scale, int* ids, float* wts, void* stream) {
    if (rows <= 0) return 0;
    if (E < 1 || E > 1024 || top < 1 || top > E || n_splits < 1) return CML_ERR_BAD_SIZE;
    if (n_groups < 1 || E % n_groups || keep_groups < 1 || keep_groups > n_groups) return CML_ERR_BAD_SIZE;
    const bool separate = correction != nullptr || n_groups > 1;
    const size_t smem = (size_t)4 * (separate ? 2 * E + n_groups : E) * sizeof(float);
    launch_pdl(route_topk_kernel, dim3((rows + 3) / 4), dim3(128), smem, (cudaStream_t)stream, logits, ld,
               n_splits, split_stride, rows, E, top, score_mode, renorm, correction, n_groups, keep_groups, weight_scale, ids, wts);
    return cml_launch_status();
}

// Block e walks all pairs in order and numbers those that chose expert e: a stable counting sort, one block
// per expert, no atomics.
__global__ void __launch_bounds__(256) expert_rank_kernel(const int* __restrict__ ids, int pairs, int* __restrict__ rank,
                                                          int* __restrict__ counts) {
    __shared__ int warp_tot[8];
    pdl_wait();
    pdl_launch_dependents();
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int running = 0;
    for (int base = 0; base < pairs; base += 256) {
        const int p = base + threadIdx.x;
        const bool flag = p < pairs && ids[p] == e;
        const unsigned b = __ballot_sync(0xffffffffu, flag);
        if (lane == 0) warp_tot[warp] = __popc(b);
        __syncthreads();
        int before = 0, all = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            before += w < warp ? warp_tot[w] : 0;
            all += warp_tot[w];
        }
        if (flag) rank[p] = running + before + __popc(b & ((1u << lane) - 1u));
        running += all;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = running;
}

// offsets[e] = pairs of experts before e; tile_first[e] = tiles of tile_rows rows of experts before e (both E + 1 long).
__global__ void __launch_bounds__(1024) expert_offsets_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                                              int* __restrict__ tile_first, int tile_rows) {
    __shared__ int s_cnt[1024], s_tile[1024];
    pdl_wait();
    pdl_launch_dependents();
    const int t = threadIdx.x;
    const int c = t < E ? counts[t] : 0;
    s_cnt[t] = c;
    s_tile[t] = (c + tile_rows - 1) / tile_rows;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {                        // inclusive sums, doubling
        const int a = t >= d ? s_cnt[t - d] : 0, b = t >= d ? s_tile[t - d] : 0;
        __syncthreads();
        s_cnt[t] += a;
        s_tile[t] += b;
        __syncthreads();
    }
    if (t < E) {
        offsets[t + 1] = s_cnt[t];
        tile_first[t + 1] = s_tile[t];
    }
    if (t == 0) { offsets[0] = 0; tile_first[0] = 0; }
}

extern "C" int cml_expert_plan(const int* ids, int pairs, int E, int* rank, int* counts, int* offsets, int* tile_first,
                               int tile_rows, void* stream) {
    if (pairs <= 0) return 0;
    if (E < 1 || E > 1024 || tile_rows < 1) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    launch_pdl(expert_rank_kernel, dim3(E), dim3(256), 0, s, ids, pairs, rank, counts);
    launch_pdl(expert_offsets_kernel, dim3(1), dim3(1024), 0, s, (const int*)counts, E, offsets, tile_first, tile_rows);
    return cml_launch_status();
}

// xs[pos] = x[row] (* weight), pos = offsets[expert] + rank; pos_of_pair remembers pos. One block per pair.
// Experts real_experts and up are identity experts (their output is their input): nothing is copied for them.
template <typename T>
__global__ void expert_gather_kernel(const T* __restrict__ x, long ldx, int width, const int* __restrict__ ids,
                                     const float* __restrict__ wts, const int* __restrict__ rank, const int* __restrict__ offsets,
                                     int top, int scale_input, int real_experts, T* __restrict__ xs,
                                     int* __restrict__ pos_of_pair) {
    pdl_wait();
    pdl_launch_dependents();
    const int p = blockIdx.x;
    const int pos = offsets[ids[p]] + rank[p];
    if (ids[p] >= real_experts) {                               // an identity expert: no product reads its rows
        if (threadIdx.x == 0) pos_of_pair[p] = pos;
        return;
    }
    const float w = scale_input ? wts[p] : 1.0f;
    const T* src = x + (size_t)(p / top) * ldx;
    T* dst = xs + (size_t)pos * width;
    constexpr int VEC = 16 / (int)sizeof(T);
    if (width % VEC == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {          // rows in 16-byte pieces
        for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
            union { uint4 raw; T e[VEC]; } v;
            v.raw = *reinterpret_cast<const uint4*>(src + c);
            if (scale_input) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) v.e[k] = from_f32<T>(to_f32(v.e[k]) * w);
            }
            *reinterpret_cast<uint4*>(dst + c) = v.raw;
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = scale_input ? from_f32<T>(to_f32(src[c]) * w) : src[c];
    }
    if (threadIdx.x == 0) pos_of_pair[p] = pos;
}

extern "C" int cml_expert_gather(const void* x, int dtype, long ldx, int width, const int* ids, const float* wts, const int* rank,
                                 const int* offsets, int pairs, int top, int scale_input, int real_experts, void* xs, int* pos_of_pair,
                                 void* stream) {
    if (pairs <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int block = width >= 1024 ? 256 : 128;
    if (dtype == CML_DTYPE_F32)
        launch_pdl(expert_gather_kernel<float>, dim3(pairs), dim3(block), 0, s, (const float*)x, ldx, width, ids, wts, rank, offsets,
                   top, scale_input, real_experts, (float*)xs, pos_of_pair);
    else if (dtype == CML_DTYPE_BF16)
        launch_pdl(expert_gather_kernel<bf16>, dim3(pairs), dim3(block), 0, s, (const bf16*)x, ldx, width, ids, wts, rank, offsets,
                   top, scale_input, real_experts, (bf16*)xs, pos_of_pair);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}

// The grouped product on the CUDA cores, float accumulation (the true 32-bit path, and the bfloat16 path's
// fallback): a block owns 64 rows of one expert's stretch by 64 output features; a thread 4 x 4 of them.
// W [E, N, K] (and W2 the same for the gated form). GATED: out = silu(A Wg^T) * (A Wu^T) in the compute type;
// else out float = A W^T.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) expert_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, const T* __restrict__ W2,
                                                          void* __restrict__ out, int N, int K, int E,
                                                          const int* __restrict__ offsets, const int* __restrict__ tile_first,
                                                          const GateAct act) {
    __shared__ float As[EX_TK][EX_TM + 4];
    __shared__ float Ws[GATED ? 2 : 1][EX_TK][EX_TN + 4];
    pdl_wait();
    pdl_launch_dependents();
    const int tile = blockIdx.y;
    if (tile >= tile_first[E]) return;
    int lo = 0, hi = E;                                         // the expert whose tiles hold this one
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (tile_first[mid] <= tile) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int row0 = offsets[e] + (tile - tile_first[e]) * EX_TM, row_end = offsets[e + 1];
    const int n0 = blockIdx.x * EX_TN;
    const T* We = W + (size_t)e * N * K;
    const T* We2 = GATED ? W2 + (size_t)e * N * K : nullptr;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;    // 16 x 16 threads: ty rows, tx columns
    float acc[4][4], acc2[GATED ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (GATED) acc2[i][j] = 0.f; }
    // loads: thread t takes element (t / 16 + 16 * u, t % 16) of a 64 x 16 tile, u = 0..3
    const int lk = threadIdx.x & 15, lr = threadIdx.x >> 4;
    for (int k0 = 0; k0 < K; k0 += EX_TK) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int rr = lr + 16 * u, kk = k0 + lk;
            const int row = row0 + rr, n = n0 + rr;
            As[lk][rr] = (row < row_end && kk < K) ? to_f32(A[(size_t)row * K + kk]) : 0.f;
            Ws[0][lk][rr] = (n < N && kk < K) ? to_f32(We[(size_t)n * K + kk]) : 0.f;
            if (GATED) Ws[1][lk][rr] = (n < N && kk < K) ? to_f32(We2[(size_t)n * K + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < EX_TK; ++kk) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { b[j] = Ws[0][kk][tx * 4 + j]; if (GATED) b2[j] = Ws[1][kk][tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + ty * 4 + i;
        if (row >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GATED) {
                const float g = acc[i][j];
                ((T*)out)[(size_t)row * N + n] = from_f32<T>(gate_act(g, acc2[i][j], act));
            } else {
                ((float*)out)[(size_t)row * N + n] = acc[i][j];
            }
        }
    }
}

extern "C" int cml_expert_gemm(const void* A, const void* W, const void* W2, int dtype, void* out, int pairs, int N, int K, int E,
                               const int* offsets, const int* tile_first, void* stream) {
    if (pairs <= 0) return 0;
    const int max_tiles = (pairs + EX_TM - 1) / EX_TM + (E < pairs ? E : pairs);
    dim3 grid((N + EX_TN - 1) / EX_TN, max_tiles);
    if (max_tiles > 65535) return CML_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
#define EG_CASE(T_, G_)                                                                                                     \
    launch_pdl(expert_gemm_kernel<T_, G_>, grid, dim3(256), 0, s, (const T_*)A, (const T_*)W, (const T_*)W2, out, N, K, E, offsets, \
               tile_first, cml_gate_act_now)
    if (dtype == CML_DTYPE_F32) { if (W2) EG_CASE(float, true); else EG_CASE(float, false); }
    else if (dtype == CML_DTYPE_BF16) { if (W2) EG_CASE(bf16, true); else EG_CASE(bf16, false); }
    else return CML_ERR_BAD_DTYPE;
#undef EG_CASE
    return cml_launch_status();
}

// out[row] = sum over splits of shared[split][row] + sum over the row's choices, in their order, of y[pos] (* weight).
// A choice of an identity expert (ids >= real_experts; `ids` may be null: there are none) adds the row itself
// (`same` [rows, hidden], float or the compute type) times its weight.
template <typename TS>
__global__ void expert_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of_pair, const float* __restrict__ wts,
                                      int top, int scale_output, const float* __restrict__ shared, int shared_splits,
                                      long shared_stride, const int* __restrict__ ids, int real_experts,
                                      const TS* __restrict__ same, float* __restrict__ out, int hidden) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    if ((hidden & 3) == 0) {                                    // four columns a thread, 16-byte accesses
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < shared_splits; ++s) {
                const float4 t = *reinterpret_cast<const float4*>(shared + (size_t)s * shared_stride + (size_t)r * hidden + c);
                v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            }
            for (int k = 0; k < top; ++k) {
                const int p = r * top + k;
                const bool ident = ids != nullptr && ids[p] >= real_experts;
                float4 t;
                if (ident) {
                    const TS* sr = same + (size_t)r * hidden + c;
                    t = make_float4(to_f32(sr[0]), to_f32(sr[1]), to_f32(sr[2]), to_f32(sr[3]));
                } else {
                    t = *reinterpret_cast<const float4*>(y + (size_t)pos_of_pair[p] * hidden + c);
                }
                const float w = (scale_output || ident) ? wts[p] : 1.0f;
                v.x += t.x * w; v.y += t.y * w; v.z += t.z * w; v.w += t.w * w;
            }
            *reinterpret_cast<float4*>(out + (size_t)r * hidden + c) = v;
        }
        return;
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < shared_splits; ++s) v += shared[(size_t)s * shared_stride + (size_t)r * hidden + c];
        for (int k = 0; k < top; ++k) {
            const int p = r * top + k;
            const bool ident = ids != nullptr && ids[p] >= real_experts;
            const float t = ident ? to_f32(same[(size_t)r * hidden + c]) : y[(size_t)pos_of_pair[p] * hidden + c];
            v += (scale_output || ident) ? t * wts[p] : t;
        }
        out[(size_t)r * hidden + c] = v;
    }
}

extern "C" int cml_expert_combine(const float* y, const int* pos_of_pair, const float* wts, int top, int scale_output,
                                  const float* shared, int shared_splits, long shared_stride, const int* ids, int real_experts,
                                  const void* same, int same_dtype, float* out, int rows, int hidden, void* stream) {
    if (rows <= 0) return 0;
    if (ids != nullptr && same == nullptr) return CML_ERR_BAD_SIZE;
    const dim3 block(hidden >= 1024 ? 256 : 128);
    if (same_dtype == CML_DTYPE_BF16)
        launch_pdl(expert_combine_kernel<bf16>, dim3(rows), block, 0, (cudaStream_t)stream, y, pos_of_pair, wts, top,
                   scale_output, shared, shared ? shared_splits : 0, shared_stride, ids, real_experts, (const bf16*)same, out, hidden);
    else
        launch_pdl(expert_combine_kernel<float>, dim3(rows), block, 0, (cudaStream_t)stream, y, pos_of_pair, wts, top,
                   scale_output, shared, shared ? shared_splits : 0, shared_stride, ids, real_experts, (const float*)same, out, hidden);
    return cml_launch_status();
}
