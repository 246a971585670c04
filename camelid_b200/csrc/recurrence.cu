// Recurrent mixers with a matrix state per head: S [key_dim, value_dim] in float, carried from
// token to token for each sequence.
//
//   gated delta rule (one decay per key channel, or one per head):  S <- diag(g) S;  u = beta (v - S^T k);
//                                                  S <- S + k u^T;  o = S^T q
//   matrix memory with exponential gates:          m' = max(f + m, i);
//                                                  S <- e^(f + m - m') S + e^(i - m') k v^T  (n likewise with k alone);
//                                                  o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)
//
//   retention (a fixed decay per head):            S <- d S + k v^T;  o = S^T q
//
// All are independent per column of S: eight threads of a warp share one column (a slice of
// the key axis each, in registers) of one (sequence, head) and walk the sequence's new tokens
// in order, so a prompt's rows and the same rows fed one by one are summed in the same order.
// The matrix memory keeps n as one more column (whose v is 1) and a copy of m per column, so
// that no thread reads what another writes. q, k, gates of a few tokens at a time are staged
// in shared memory by the whole block.
//
// Before them: the short causal convolution with SiLU and the unit norm of q and k for the
// delta rule. After them: the per-head RMS norm with weight and sigmoid gate.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoid_f(float x) { return x < 0.f ? x - log1pf(expf(x)) : -log1pf(expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------------------------
// Short convolution + SiLU (+ unit norm). `proj` [rows, ld] holds, from column 0, the q
// channels (qk_heads x key_dim), the k channels (the same) and the v channels (heads x
// value_dim) before the convolution; `conv_w` [channels, taps] float, the last tap the current
// token's; `state` [slots, taps - 1, channels] the inputs of the tokens before the step.
// A warp owns one (row, head of q | k | v). q and k become x / sqrt(sum x^2 + 1e-6), q times
// q_scale. out [rows, channels] float. With `update_state` (steps in which every sequence brings
// one row) the warp also moves its channels of the state on by that row; otherwise a later
// launch replaces the state.
__global__ void conv_unit_kernel(const float* __restrict__ proj, long ld, const float* __restrict__ conv_w,
                                 float* __restrict__ state, int update_state, const int* __restrict__ row_seq,
                                 const int* __restrict__ row_pos, const int* __restrict__ seq_row0,
                                 const int* __restrict__ seq_slot, float* __restrict__ out, int rows, int qk_heads,
                                 int heads, int key_dim, int value_dim, int taps, float q_scale,
                                 const float* __restrict__ decay_in, long ldd, const float* __restrict__ a_log,
                                 const float* __restrict__ dt_bias, float* __restrict__ decay_out, int decay_dim) {
    pdl_wait();
    pdl_launch_dependents();
    const int units = 2 * qk_heads + heads + (decay_in ? heads : 0);
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * units) return;
    const int r = warp / units, u = warp % units;
    if (u >= 2 * qk_heads + heads) {
        // the decays of one (row, head), once for all the scan's blocks of that head:
        // g = exp(-exp(a_log[head]) softplus(x + dt_bias))
        const int hd = u - 2 * qk_heads - heads;
        const float rate = expf(a_log[hd]);
        for (int d = lane; d < decay_dim; d += 32) {            // decay_dim: key_dim (a decay per channel) or 1 (per head)
            const float x = decay_in[(size_t)r * ldd + hd * decay_dim + d] + dt_bias[hd * decay_dim + d];
            decay_out[((size_t)r * heads + hd) * decay_dim + d] = expf(-rate * softplus_f(x));
        }
        return;
    }
    const int channels = 2 * qk_heads * key_dim + heads * value_dim;
    int c0, n;
    if (u < 2 * qk_heads) { c0 = u * key_dim; n = key_dim; }
    else { c0 = 2 * qk_heads * key_dim + (u - 2 * qk_heads) * value_dim; n = value_dim; }
    const int s = row_seq[r], pos = row_pos[r], inside = r - seq_row0[s];
    float* st = state + (size_t)seq_slot[s] * (taps - 1) * channels;
    float ss = 0.f;
    // A lane's channels eight at a time, tap by tap: the eight loads of a tap are unconditional (of a valid
    // place) and in flight together; nothing is stored until every tap has been read.
    for (int base = c0; base < c0 + n; base += 256) {
        float acc[8];
        int cc[8];
        bool ok[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int c = base + lane + 32 * e;
            ok[e] = c < c0 + n;
            cc[e] = ok[e] ? c : c0;
            acc[e] = 0.f;
        }
        const int ne = min(8, (c0 + n - base + 31) / 32);  // groups of 32 channels that are there at all (the same for the warp)
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;                 // tokens before this one
            if (back > pos) continue;                      // before the sequence's start
            const float* src = back <= inside ? proj + (size_t)(r - back) * ld : st + (size_t)(taps - 1 + inside - back) * channels;
            float x[8], w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (e < ne) { x[e] = src[cc[e]]; w[e] = conv_w[(size_t)cc[e] * taps + j]; }
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (e < ne) acc[e] = fmaf(w[e], x[e], acc[e]);
        }
        if (update_state && taps > 1) {                    // one row per sequence: drop the oldest input, keep this one
            for (int j = 0; j + 2 < taps; ++j) {
                float t[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) t[e] = st[(size_t)(j + 1) * channels + cc[e]];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (ok[e]) st[(size_t)j * channels + cc[e]] = pos + j + 2 >= taps ? t[e] : 0.f;
            }
            float t[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = proj[(size_t)r * ld + cc[e]];
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (ok[e]) st[(size_t)(taps - 2) * channels + cc[e]] = t[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (!ok[e]) continue;
            const float a = silu_f(acc[e]);
            out[(size_t)r * channels + cc[e]] = a;
            ss = fmaf(a, a, ss);
        }
    }
    if (u < 2 * qk_heads) {
        ss = warp_sum(ss);
        const float scale = (u < qk_heads ? q_scale : 1.0f) / sqrtf(ss + 1e-6f);
        __syncwarp();
        for (int c = c0 + lane; c < c0 + n; c += 32) out[(size_t)r * channels + c] *= scale;
    }
}

// decay_in (may be null) [rows, ldd] (heads x decay_dim, decay_dim = key_dim or 1): the decays' inputs; decay_out [rows, heads x decay_dim] gets
// g = exp(-exp(a_log[head]) softplus(x + dt_bias)), what the delta-rule scan multiplies its state by.
extern "C" int cml_conv_unit(const float* proj, long ld, const float* conv_w, float* state, int update_state, const int* row_seq,
                             const int* row_pos, const int* seq_row0, const int* seq_slot, float* out, int rows, int qk_heads,
                             int heads, int key_dim, int value_dim, int taps, float q_scale, const float* decay_in, long ldd,
                             const float* a_log, const float* dt_bias, float* decay_out, int decay_dim, void* stream) {
    if (rows <= 0) return 0;
    if (taps < 1 || (decay_in && decay_dim != 1 && decay_dim != key_dim)) return CML_ERR_BAD_SIZE;
    const long warps = (long)rows * (2 * qk_heads + heads + (decay_in ? heads : 0));
    launch_pdl(conv_unit_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, proj, ld, conv_w, state,
               update_state, row_seq, row_pos, seq_row0, seq_slot, out, rows, qk_heads, heads, key_dim, value_dim, taps, q_scale, decay_in, ldd,
               a_log, dt_bias, decay_out, decay_dim);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// The scans. A block of 128 threads owns 128 / NS columns of one (sequence, head); the key axis of a
// column is cut into NS slices (a power of two up to 32) of DS channels, one thread each, the NS
// threads of a column in one warp (lane = NS * column + slice), so that a dot product over the key
// axis is DS multiply-adds and a butterfly of log2 NS shuffles, always in the same order, whatever
// the step or the batch. The delta rule takes its two products
// (with k for the write, with q for the read-out) from the decayed state at once and adds the
// write's share u (k . q) to the read-out, so a token waits only for the write of the one before. The state lies column by column
// ([.., column, key channel]): a warp reads and writes whole rows of it with 16-byte accesses.
// q, k and the decays of SCAN_TOKENS tokens at a time stand in shared memory (slices padded by
// four floats against bank conflicts); the next tokens' values are fetched into registers
// while these are worked on.
//
// MODE 0, gated delta rule. in_a = qkv [rows, lda]: unit q (qk_heads x D), unit k, v (heads x Dv)
// from conv_unit_kernel; in_b [rows, ldb]: beta before the sigmoid at column b_col + head;
// in_c [rows, ldc] (heads x D, or heads with one decay per head): the decays g (decay_ready), or their input:
// g = exp(-exp(a_log[head]) softplus(x + dt_bias)).
// state [slots, heads, Dv, D]. out [rows, heads x Dv] = S^T q.
// MODE 1, matrix memory. in_a = proj [rows, lda] with q at q_col (heads x D), k at k_col, v at
// v_col (heads x Dv), gate inputs at i_col + head and f_col + head (before bias and cap).
// state [slots, heads, Dv + 1, D] (column Dv is n), state_m [slots, heads, Dv + 1] (m, one copy
// per column, so that no thread reads what another writes). out [rows, heads, Dv + 2]: S^T q per
// column, then n . q, then m after the token.
// MODE 2, retention. in_a = proj [rows, lda] with q at q_col (heads x D), k at k_col, v at v_col (heads x Dv), q and k
// turned and scaled already; vec_a [heads]: the heads' decays. state [slots, heads, Dv, D]. out [rows, heads x Dv].
#define SCAN_TOKENS 8

struct ScanParams {
    const float* in_a; long lda;
    const float* in_b; long ldb; int b_col;
    const float* in_c; long ldc;
    const float* vec_a;           // a_log [heads]            | input-gate bias [heads]
    const float* vec_b;           // dt_bias [heads x D]      | forget-gate bias [heads]
    float* state; float* state_m;
    const int* seq_row0; const int* seq_new; const int* seq_start; const int* seq_slot;
    float* out;
    int heads, qk_heads, D, Dv;
    int q_col, k_col, v_col, i_col, f_col;
    float cap, q_scale;
    int decay_ready;              // in_c holds the decays themselves (conv_unit_kernel made them)
    int decay_dim;                // D: one decay per key channel; 1: one per head (in_c and vec_b are heads x decay_dim)
};

template <int NS>
__device__ __forceinline__ float slices_sum(float v) {
#pragma unroll
    for (int sh = 1; sh < NS; sh <<= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
    return v;
}

template <int DS, int MODE, int NS>
__global__ void __launch_bounds__(128) scan_kernel(const ScanParams p) {
    constexpr int SCAN_COLS = 128 / NS;                // columns of a block
    constexpr int DPAD = NS * DS;                      // key channels a block can take
    constexpr int SL = DS == 4 ? 4 : DS + 4;           // floats of a slice in shared memory (padded against bank conflicts)
    constexpr int PER = SCAN_TOKENS * DPAD / 128;      // staged values per thread and array
    __shared__ __align__(16) float sq[SCAN_TOKENS][NS * SL], sk[SCAN_TOKENS][NS * SL], sg[MODE == 0 ? SCAN_TOKENS : 1][NS * SL];
    __shared__ float sv[SCAN_TOKENS][SCAN_COLS], s1[SCAN_TOKENS], s2[SCAN_TOKENS], skq[SCAN_TOKENS];
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x, hd = blockIdx.y;
    const int D = p.D, Dv = p.Dv, heads = p.heads;
    const int cols = MODE == 1 ? Dv + 1 : Dv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slice = lane % NS;
    const int wcol = warp * (32 / NS) + lane / NS;       // this thread's column within the block
    const int c = blockIdx.z * SCAN_COLS + wcol;
    const bool live = c < cols;
    const int d0 = slice * DS;
    const int row0 = p.seq_row0[s], n = p.seq_new[s];
    const bool fresh = p.seq_start[s] == 0;
    const size_t cell = ((size_t)p.seq_slot[s] * heads + hd) * cols + (live ? c : 0);
    float* st = p.state + cell * D;
    const bool vec = (D & 3) == 0;
    float S[DS];
#pragma unroll
    for (int i = 0; i < DS; i += 4) {
        if (live && !fresh && vec && d0 + i < D) {
            const float4 t = *reinterpret_cast<const float4*>(st + d0 + i);
            S[i] = t.x; S[i + 1] = t.y; S[i + 2] = t.z; S[i + 3] = t.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) S[i + j] = (live && !fresh && d0 + i + j < D) ? st[d0 + i + j] : 0.f;
        }
    }
    float m = 0.f;
    if (MODE == 1 && live && !fresh) m = p.state_m[cell];
    const float keep = MODE == 2 ? p.vec_a[hd] : 0.f;          // retention: the head's decay
    const int g = MODE == 0 ? hd / (heads / p.qk_heads) : hd;
    const int qc = MODE == 0 ? g * D : p.q_col + hd * D;
    const int kc = MODE == 0 ? (p.qk_heads + g) * D : p.k_col + hd * D;
    const int vc = MODE == 0 ? 2 * p.qk_heads * D + hd * Dv : p.v_col + hd * Dv;
    const float a_rate = (MODE == 0 && !p.decay_ready) ? expf(p.vec_a[hd]) : 0.f;
    const bool head_decay = MODE == 0 && p.decay_dim == 1;      // one decay per head: a number per token (s2), not a row of sg
    // staging: thread -> (token, key channel) of each array, one value of v, and the scalars
    // Nothing uses a fetched value before `stage`: a use right behind its load would hold the warp until the
    // load is back, once per round, instead of behind the tokens in between.
    float rq[PER], rk[PER], rg[MODE == 0 ? PER : 1], rv = 0.f, r1 = 0.f, r2 = 0.f;
    float bias[MODE == 0 ? PER : 1];                   // dt_bias of the channels this thread stages (the same every round)
    if (MODE == 0 && !p.decay_ready) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int d = (threadIdx.x + 128 * e) % DPAD;
            bias[e] = p.vec_b[head_decay ? hd : hd * D + (d < D ? d : 0)];
        }
    }
    auto fetch = [&](int t0) {
        const int nt = min(SCAN_TOKENS, n - t0);
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = threadIdx.x + 128 * e, t = idx / DPAD, d = idx % DPAD;
            const bool ok = t < nt && d < D;
            const size_t r = (size_t)(row0 + t0 + (ok ? t : 0));
            const int dd = ok ? d : 0;
            rq[e] = p.in_a[r * p.lda + qc + dd];
            rk[e] = p.in_a[r * p.lda + kc + dd];
            if (MODE == 0 && !head_decay) rg[e] = p.in_c[r * p.ldc + hd * D + dd];
        }
        if (threadIdx.x < SCAN_TOKENS * SCAN_COLS) {
            const int t = threadIdx.x / SCAN_COLS, cc = blockIdx.z * SCAN_COLS + threadIdx.x % SCAN_COLS;
            const bool ok = t < nt && cc < Dv;
            rv = p.in_a[(size_t)(row0 + t0 + (ok ? t : 0)) * p.lda + vc + (ok ? cc : 0)];
        }
        if (threadIdx.x < SCAN_TOKENS) {
            const size_t r = (size_t)(row0 + t0 + (threadIdx.x < nt ? threadIdx.x : 0));
            if (MODE == 0) {
                r1 = p.in_b[r * p.ldb + p.b_col + hd];
                if (head_decay) r2 = p.in_c[r * p.ldc + hd];
            } else if (MODE == 1) { r1 = p.in_a[r * p.lda + p.i_col + hd]; r2 = p.in_a[r * p.lda + p.f_col + hd]; }
        }
        // The loads stay here, ahead of the tokens that are worked on meanwhile: without this the compiler moves
        // them down to their first use, where the warp would wait for them. (No instruction is emitted.)
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            asm volatile("" : "+f"(rq[e]), "+f"(rk[e]));
            if (MODE == 0) asm volatile("" : "+f"(rg[e]));
        }
        asm volatile("" : "+f"(rv), "+f"(r1), "+f"(r2));
    };
    auto stage = [&]() {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = threadIdx.x + 128 * e, t = idx / DPAD, d = idx % DPAD;
            const int at = (d / DS) * SL + d % DS;
            const bool in = d < D;                     // channels beyond D stay out of every sum
            sq[t][at] = in ? (MODE == 1 ? rq[e] * p.q_scale : rq[e]) : 0.f;
            sk[t][at] = in ? rk[e] : 0.f;
            if (MODE == 0 && !head_decay) sg[t][at] = p.decay_ready ? rg[e] : expf(-a_rate * softplus_f(rg[e] + bias[e]));
        }
        if (threadIdx.x < SCAN_TOKENS * SCAN_COLS) {
            const int cc = blockIdx.z * SCAN_COLS + threadIdx.x % SCAN_COLS;
            sv[threadIdx.x / SCAN_COLS][threadIdx.x % SCAN_COLS] = cc < Dv ? rv : ((MODE == 1 && cc == Dv) ? 1.0f : 0.f);   // the column of n has v = 1
        }
        if (threadIdx.x < SCAN_TOKENS) {
            if (MODE == 0) {
                s1[threadIdx.x] = sigmoid_f(r1);
                if (head_decay) s2[threadIdx.x] = p.decay_ready ? r2 : expf(-a_rate * softplus_f(r2 + p.vec_b[hd]));
            } else if (MODE == 1) {
                s1[threadIdx.x] = p.cap * tanhf((r1 + p.vec_a[hd]) / p.cap);
                s2[threadIdx.x] = logsigmoid_f(p.cap * tanhf((r2 + p.vec_b[hd]) / p.cap));
            }
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < n; t0 += SCAN_TOKENS) {
        const int nt = min(SCAN_TOKENS, n - t0);
        __syncthreads();                               // the tokens before are done with the staged values
        stage();
        __syncthreads();
        if (MODE == 0) {
            // k . q of every staged token, the same for all columns: warp w takes tokens 2w and 2w + 1
#pragma unroll
            for (int tt = 0; tt < SCAN_TOKENS / 4; ++tt) {
                const int t = warp * (SCAN_TOKENS / 4) + tt;
                float a = 0.f;
                for (int d = lane; d < DPAD; d += 32) {
                    const int at = (d / DS) * SL + d % DS;
                    a = fmaf(sk[t][at], sq[t][at], a);
                }
                a = warp_sum(a);
                if (lane == 0) skq[t] = a;
            }
            __syncthreads();
        }
        if (t0 + SCAN_TOKENS < n) fetch(t0 + SCAN_TOKENS);
        // Gated delta rule, one token. With S' = diag(g) S both products S'^T k and S'^T q are taken at once (two
        // butterflies side by side), and since the state after the write is S' + k u^T, the read-out is
        // S'^T q + u (k . q): the only thing the next token waits for is the write itself.
        auto delta_token = [&](int t) {
            const float* kq = &sk[t][slice * SL];
            const float* qq = &sq[t][slice * SL];
            const float* gg = &sg[t][slice * SL];
            const float vcol = sv[t][wcol];
            float kr[DS];
            float d4[4] = {0.f, 0.f, 0.f, 0.f}, o4[4] = {0.f, 0.f, 0.f, 0.f};       // four chains each, always in this order
            if (head_decay) {
                const float gh = s2[t];
#pragma unroll
                for (int i = 0; i < DS; ++i) S[i] *= gh;
            } else {
#pragma unroll
                for (int i = 0; i < DS; i += 4) {
                    const float4 gv = *reinterpret_cast<const float4*>(gg + i);
                    S[i] *= gv.x; S[i + 1] *= gv.y; S[i + 2] *= gv.z; S[i + 3] *= gv.w;
                }
            }
#pragma unroll
            for (int i = 0; i < DS; i += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kq + i);
                const float4 qv = *reinterpret_cast<const float4*>(qq + i);
                kr[i] = kv.x; kr[i + 1] = kv.y; kr[i + 2] = kv.z; kr[i + 3] = kv.w;
                d4[0] = fmaf(S[i], kv.x, d4[0]); d4[1] = fmaf(S[i + 1], kv.y, d4[1]);
                d4[2] = fmaf(S[i + 2], kv.z, d4[2]); d4[3] = fmaf(S[i + 3], kv.w, d4[3]);
                o4[0] = fmaf(S[i], qv.x, o4[0]); o4[1] = fmaf(S[i + 1], qv.y, o4[1]);
                o4[2] = fmaf(S[i + 2], qv.z, o4[2]); o4[3] = fmaf(S[i + 3], qv.w, o4[3]);
            }
            float dk = (d4[0] + d4[1]) + (d4[2] + d4[3]), dq = (o4[0] + o4[1]) + (o4[2] + o4[3]);
#pragma unroll
            for (int sh = 1; sh < NS; sh <<= 1) {
                const float a = __shfl_xor_sync(0xffffffffu, dk, sh), b = __shfl_xor_sync(0xffffffffu, dq, sh);
                dk += a;
                dq += b;
            }
            const float u = s1[t] * (vcol - dk);
#pragma unroll
            for (int i = 0; i < DS; ++i) S[i] = fmaf(kr[i], u, S[i]);
            if (live && slice == 0) p.out[(size_t)(row0 + t0 + t) * heads * Dv + hd * Dv + c] = fmaf(u, skq[t], dq);
        };
        if constexpr (MODE == 0) {
            if (nt == SCAN_TOKENS) {        // a whole round unrolled: the next tokens' loads and this one's read-out overlap
#pragma unroll
                for (int t = 0; t < SCAN_TOKENS; ++t) delta_token(t);
            } else {
                for (int t = 0; t < nt; ++t) delta_token(t);
            }
        } else if constexpr (MODE == 2) {
            // Retention, one token: S = d S + k v, then the read-out from the new state; four chains, always in this order.
            auto retention_token = [&](int t) {
                const float* kq = &sk[t][slice * SL];
                const float* qq = &sq[t][slice * SL];
                const float vcol = sv[t][wcol];
                float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < DS; i += 4) {
                    const float4 kv = *reinterpret_cast<const float4*>(kq + i), qv = *reinterpret_cast<const float4*>(qq + i);
                    S[i] = fmaf(keep, S[i], vcol * kv.x); S[i + 1] = fmaf(keep, S[i + 1], vcol * kv.y);
                    S[i + 2] = fmaf(keep, S[i + 2], vcol * kv.z); S[i + 3] = fmaf(keep, S[i + 3], vcol * kv.w);
                    o4[0] = fmaf(S[i], qv.x, o4[0]); o4[1] = fmaf(S[i + 1], qv.y, o4[1]);
                    o4[2] = fmaf(S[i + 2], qv.z, o4[2]); o4[3] = fmaf(S[i + 3], qv.w, o4[3]);
                }
                const float o = slices_sum<NS>((o4[0] + o4[1]) + (o4[2] + o4[3]));
                if (live && slice == 0) p.out[(size_t)(row0 + t0 + t) * heads * Dv + hd * Dv + c] = o;
            };
            if (nt == SCAN_TOKENS) {
#pragma unroll
                for (int t = 0; t < SCAN_TOKENS; ++t) retention_token(t);
            } else {
                for (int t = 0; t < nt; ++t) retention_token(t);
            }
        } else {
            for (int t = 0; t < nt; ++t) {
                const float* kq = &sk[t][slice * SL];
                const float* qq = &sq[t][slice * SL];
                const float vcol = sv[t][wcol];
                float o = 0.f;
                const float fm = s2[t] + m;
                const float m_new = fmaxf(fm, s1[t]);
                const float a = expf(fm - m_new);
                const float bv = expf(s1[t] - m_new) * vcol;
                m = m_new;
                float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < DS; i += 4) {
                    const float4 kv = *reinterpret_cast<const float4*>(kq + i), qv = *reinterpret_cast<const float4*>(qq + i);
                    S[i] = fmaf(a, S[i], bv * kv.x); S[i + 1] = fmaf(a, S[i + 1], bv * kv.y);
                    S[i + 2] = fmaf(a, S[i + 2], bv * kv.z); S[i + 3] = fmaf(a, S[i + 3], bv * kv.w);
                    o4[0] = fmaf(S[i], qv.x, o4[0]); o4[1] = fmaf(S[i + 1], qv.y, o4[1]);
                    o4[2] = fmaf(S[i + 2], qv.z, o4[2]); o4[3] = fmaf(S[i + 3], qv.w, o4[3]);
                }
                o = slices_sum<NS>((o4[0] + o4[1]) + (o4[2] + o4[3]));
                if (live && slice == 0) {
                    float* orow = p.out + ((size_t)(row0 + t0 + t) * heads + hd) * (Dv + 2);
                    orow[c] = o;
                    if (c == Dv) orow[Dv + 1] = m;
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DS; i += 4) {
            if (vec && d0 + i < D) {
                *reinterpret_cast<float4*>(st + d0 + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (d0 + i + j < D) st[d0 + i + j] = S[i + j];
            }
        }
        if (MODE == 1 && slice == 0) p.state_m[cell] = m;
    }
}

// Eight slices per column: with 16 or 32 (more and lighter warps for a lone prompt) the staging of q and k, which every
// block repeats, weighs as much as the shorter sums save, and a prompt ran no faster.
#define SCAN_SLICES 8

template <int MODE>
static int launch_scan(const ScanParams& p, int n_seqs, cudaStream_t s) {
    if (n_seqs <= 0) return 0;
    if (p.D < 1 || p.D > 256 || p.Dv < 1) return CML_ERR_BAD_SIZE;
    const int cols = MODE == 1 ? p.Dv + 1 : p.Dv;
    constexpr int block_cols = 128 / SCAN_SLICES;
    dim3 grid(n_seqs, p.heads, (cols + block_cols - 1) / block_cols);
#define SCAN_CASE(DS_)                                                                    \
    if (p.D <= SCAN_SLICES * DS_) {                                                       \
        launch_pdl(scan_kernel<DS_, MODE, SCAN_SLICES>, grid, dim3(128), 0, s, p);        \
        return cml_launch_status();                                                       \
    }
    SCAN_CASE(4) SCAN_CASE(8) SCAN_CASE(16) SCAN_CASE(32)
#undef SCAN_CASE
    return CML_ERR_BAD_SIZE;
}

extern "C" int cml_delta_scan(const float* qkv, long ldq, const float* beta_in, long ldb, int beta_col, const float* decay_in,
                              long ldd, const float* a_log, const float* dt_bias, float* state, const int* seq_row0,
                              const int* seq_new, const int* seq_start, const int* seq_slot, float* out, int n_seqs, int heads,
                              int qk_heads, int D, int Dv, int decay_ready, int decay_dim, void* stream) {
    if (qk_heads < 1 || heads % qk_heads || (decay_dim != 1 && decay_dim != D)) return CML_ERR_BAD_SIZE;
    ScanParams p = {};
    p.in_a = qkv; p.lda = ldq; p.in_b = beta_in; p.ldb = ldb; p.b_col = beta_col; p.in_c = decay_in; p.ldc = ldd;
    p.vec_a = a_log; p.vec_b = dt_bias; p.state = state; p.state_m = nullptr;
    p.seq_row0 = seq_row0; p.seq_new = seq_new; p.seq_start = seq_start; p.seq_slot = seq_slot; p.out = out;
    p.heads = heads; p.qk_heads = qk_heads; p.D = D; p.Dv = Dv; p.decay_ready = decay_ready; p.decay_dim = decay_dim;
    return launch_scan<0>(p, n_seqs, (cudaStream_t)stream);
}

extern "C" int cml_memory_scan(const float* proj, long ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                               const float* i_bias, const float* f_bias, float cap, float q_scale, float* state,
                               float* state_m, const int* seq_row0, const int* seq_new, const int* seq_start,
                               const int* seq_slot, float* out, int n_seqs, int heads, int D, int Dv, void* stream) {
    ScanParams p = {};
    p.in_a = proj; p.lda = ld; p.vec_a = i_bias; p.vec_b = f_bias; p.state = state; p.state_m = state_m;
    p.seq_row0 = seq_row0; p.seq_new = seq_new; p.seq_start = seq_start; p.seq_slot = seq_slot; p.out = out;
    p.heads = heads; p.qk_heads = heads; p.D = D; p.Dv = Dv;
    p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.i_col = i_col; p.f_col = f_col; p.cap = cap; p.q_scale = q_scale;
    return launch_scan<1>(p, n_seqs, (cudaStream_t)stream);
}

extern "C" int cml_retention_scan(const float* proj, long ld, int q_col, int k_col, int v_col, const float* decay, float* state,
                                  const int* seq_row0, const int* seq_new, const int* seq_start, const int* seq_slot,
                                  float* out, int n_seqs, int heads, int D, int Dv, void* stream) {
    ScanParams p = {};
    p.in_a = proj; p.lda = ld; p.vec_a = decay; p.state = state; p.state_m = nullptr;
    p.seq_row0 = seq_row0; p.seq_new = seq_new; p.seq_start = seq_start; p.seq_slot = seq_slot; p.out = out;
    p.heads = heads; p.qk_heads = heads; p.D = D; p.Dv = Dv;
    p.q_col = q_col; p.k_col = k_col; p.v_col = v_col; p.q_scale = 1.0f;
    return launch_scan<2>(p, n_seqs, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------
// Rotation of heads inside float rows, in place: x [rows, ld] holds `heads` heads of D channels from column col0; the
// first rot_dim channels of every head are turned by angle = position * inv_freq[i] (pairing 1: channels (2i, 2i + 1);
// 0: channels (i, i + rot_dim / 2)), sines and cosines times `amp`; then heads from number `scaled_from` on are
// multiplied by `scale` (all their channels). A warp owns one (row, head); both members of a pair are read before
// either is written.
__global__ void rotate_rows_kernel(float* __restrict__ x, long ld, int col0, int rows, int heads, int D, int rot_dim,
                                   int pairing, const float* __restrict__ inv_freq, float amp, const int* __restrict__ row_pos,
                                   int scaled_from, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * heads) return;
    const int r = warp / heads, hd = warp % heads;
    float* h = x + (size_t)r * ld + col0 + (size_t)hd * D;
    const float pos = (float)row_pos[r];
    const float mul = hd >= scaled_from ? scale : 1.0f;
    const int half = rot_dim / 2;
    for (int i = lane; i < half; i += 32) {
        const int a = pairing ? 2 * i : i, b = pairing ? 2 * i + 1 : i + half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        sn *= amp; cs *= amp;
        const float u = h[a], v = h[b];
        h[a] = (u * cs - v * sn) * mul;
        h[b] = (v * cs + u * sn) * mul;
    }
    if (mul != 1.0f)
        for (int c = rot_dim + lane; c < D; c += 32) h[c] *= mul;
}

extern "C" int cml_rotate_rows(float* x, long ld, int col0, int rows, int heads, int D, int rot_dim, int pairing,
                               const float* inv_freq, float amp, const int* row_pos, int scaled_from, float scale, void* stream) {
    if (rows <= 0 || heads <= 0) return 0;
    if (rot_dim < 0 || rot_dim > D || (rot_dim & 1)) return CML_ERR_BAD_SIZE;
    const long warps = (long)rows * heads;
    launch_pdl(rotate_rows_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, (cudaStream_t)stream, x, ld, col0, rows, heads,
               D, rot_dim, pairing, inv_freq, amp, row_pos, scaled_from, scale);
    return cml_launch_status();
}

// ------------------------------------------------------------------------------------
// After a scan: per (row, head) o = raw / den (den = max(|n . q|, exp(-m)) + 1e-6 where the
// raw rows carry them, else 1), y = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) (or * silu(gate)), written in
// the compute type for the output projection. A warp owns one (row, head). raw [rows, heads, ldh]
// with ldh = Dv (+ 2 with a denominator); w [Dv] shared by the heads (w_head_stride 0) or
// [heads x Dv]; gate [rows, ldg] at column gate_col + head * Dv.
template <typename TO>
__global__ void head_norm_gate_kernel(const float* __restrict__ raw, int ldh, int with_den, const float* __restrict__ w,
                                      int w_head_stride, const float* __restrict__ gate, long ldg, int gate_col,
                                      TO* __restrict__ out, int rows, int heads, int Dv, float eps, int gate_silu) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * heads) return;
    const int r = warp / heads, hd = warp % heads;
    const float* x = raw + ((size_t)r * heads + hd) * ldh;
    float inv = 1.0f;
    if (with_den) inv = 1.0f / (fmaxf(fabsf(x[Dv]), expf(-x[Dv + 1])) + 1e-6f);
    float ss = 0.f;
    for (int c = lane; c < Dv; c += 32) {
        const float o = x[c] * inv;
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float scale = inv / sqrtf(ss / (float)Dv + eps);
    const float* wv = w ? w + (size_t)hd * w_head_stride : nullptr;      // null: a norm without weight
    const float* gt = gate + (size_t)r * ldg + gate_col + hd * Dv;
    TO* o = out + ((size_t)r * heads + hd) * Dv;
    for (int c = lane; c < Dv; c += 32) o[c] = from_f32<TO>(x[c] * scale * (wv ? wv[c] : 1.0f) * (gate_silu ? silu_f(gt[c]) : sigmoid_f(gt[c])));
}

extern "C" int cml_head_norm_gate(const float* raw, int ldh, int with_den, const float* w, int w_head_stride, const float* gate,
                                  long ldg, int gate_col, void* out, int out_dtype, int rows, int heads, int Dv, float eps,
                                  int gate_silu, void* stream) {
    if (rows <= 0) return 0;
    const long warps = (long)rows * heads;
    dim3 grid((unsigned)((warps + 3) / 4));
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == CML_DTYPE_F32)
        launch_pdl(head_norm_gate_kernel<float>, grid, dim3(128), 0, s, raw, ldh, with_den, w, w_head_stride, gate, ldg, gate_col,
                   (float*)out, rows, heads, Dv, eps, gate_silu);
    else if (out_dtype == CML_DTYPE_BF16)
        launch_pdl(head_norm_gate_kernel<bf16>, grid, dim3(128), 0, s, raw, ldh, with_den, w, w_head_stride, gate, ldg, gate_col,
                   (bf16*)out, rows, heads, Dv, eps, gate_silu);
    else
        return CML_ERR_BAD_DTYPE;
    return cml_launch_status();
}
