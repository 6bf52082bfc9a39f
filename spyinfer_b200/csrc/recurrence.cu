// Linear recurrences over a matrix state per (request, head), carried from token to token in 32-bit:
//   * the gated matrix memory (mLSTM):       S = a S + b k v^T,  n = a n + b k,  o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
//                                            with log gates i, f, the running maximum m' = max(f + m, i) (m starts at 0),
//                                            a = exp(f + m - m'), b = exp(i - m');
//   * the generalised delta rule:            S = diag(w) S - (r u)(u^T S) + k v^T,  o = S^T q,  u = k / sqrt(sum k^2 + 1e-6),
//                                            both terms reading the old S, w a decay and r a removal rate per key channel;
//   * gated linear attention:                S = diag(a) S + k v^T,  o = S^T q,  a = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau)
//                                            a decay per key channel from the pre-activation z;
// and what follows them: each head's output divided by its root mean square, times a weight, times a gate (sigmoid or SiLU).
//
// A block owns a tile of value columns of one (request, head) (32, 16 or 8 of them: whatever gives the SMs a block each) and
// walks the request's tokens of this step in order, with its part of S in registers.  The columns of S do not depend on one
// another, so the tiles of a head run side by side; the vector n and the maximum m, which all tiles of a head need, are
// kept and updated by each tile for itself (dk + 1 numbers for every 8 columns in the state record: no tile ever reads
// what another writes, whenever their blocks happen to run).  Two kernels: one for steps with prompt portions (scan_kernel),
// whose arithmetic for a token does not depend on where a portion starts or ends, and one for steps in which every request
// brings one token (scan_decode_kernel: `longest` = 1), whose sums over a column's rows run in another order.
//
// Inputs are columns of one 32-bit activation matrix `proj` [T, ld] (the fused projection of the mixer's input).
#include "common.cuh"

SPY_MODULE(spy_recurrence)

constexpr int CT = 32;   // value columns a block of the decode kernel owns, and the widest tile of the other

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float log_sigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct ScanArgs {
    const float* proj;      // [T, ld]
    long long ld;
    int off_q, off_k, off_v, off_x1, off_x2;   // columns of q (or r), k, v; mLSTM: i and f pre-activations; delta: the removal rate's pre-activation (x2 unused)
    const float* extra;     // delta, gated linear attention: the decay's pre-activation [T, H * dk]
    const float* bias1;     // mLSTM: bias of i [H];   delta: bias of the removal rate [H * dk]
    const float* bias2;     // mLSTM: bias of f [H];   delta: the decay's offset [H * dk];   gated linear attention: the decay's bias [H * dk]
    float* state;           // [slots, H, record]
    long long record;       // floats a head: mLSTM dk * dv + (dk + 1) for every 8 columns (padded to 4); delta dk * dv
    int num_slots;
    const int* q_start;     // [S + 1]
    const int* state_slot;  // [S]
    float* out;             // [T, H * dv]
    int H, dk, dv;
    float q_scale, cap;     // cap: mLSTM: the gates' cap;   gated linear attention: 1 / tau
    int* status;
};

constexpr int THREADS = 256;      // 8 warps; warp w owns the columns 4w .. 4w + 3 of the tile, lane = 4 * (row group) + (column of the four)

// A thread keeps its part of S in registers for the whole kernel: NR consecutive rows (row group rg owns the rows
// rg * NR .. rg * NR + NR - 1; 8 * NR >= dk) of one column.  The tokens of the request are walked in chunks of TC: a
// chunk's vectors (k, q, and for the delta rule the removal rate and the decay, with their sigmoids and exponentials)
// are brought into shared memory by all threads at once, in rows of 8 * NR floats whose tail beyond dk is zero (so the
// loops over a thread's rows need no bounds); then every warp walks the chunk's tokens on its own four columns without
// a barrier (an element of S belongs to one thread, a sum over the rows is three shuffles inside the warp); the chunk's
// outputs are scaled and stored together.  The state enters and leaves through a tile in shared memory, so that global
// memory is read and written in whole rows of the tile.
// Four tokens are walked at a time: their sums over the rows are reduced together afterwards, so that the shuffles of one
// token run beside those of the others and beside the next token's rows (nothing in S waits for them).
// RG row groups share a warp's lanes (8, 16 or 32), so a warp owns 32 / RG columns and a block CTB = 8 * 32 / RG of them:
// with few requests and heads the tiles are made narrow, so that there are blocks for every SM, and a thread's rows few.
template <int MODE, int NR, int RG>   // MODE 0: gated matrix memory, 1: delta rule, 2: gated linear attention
__global__ void __launch_bounds__(THREADS, NR <= 8 ? 2 : 1) scan_kernel(ScanArgs A, int TC)
{
    constexpr int CW = 32 / RG, CTB = 8 * CW, SPB = CTB + 4;   // columns a warp and a block own; floats between the rows of the state tile in shared memory
    extern __shared__ __align__(16) float sm[];
    // Launched in plain stream order (spy_launch_in_order): it runs long on about a block an SM, and started early its
    // blocks piled up on the SMs that the product ahead left first (a prompt step was a sixth slower).
    pdl_wait();
    constexpr int KS = RG * NR;                     // floats a staged vector takes
    constexpr int V4 = NR >= 4 ? 4 : NR;           // elements a load of a thread's rows brings
    const int dk = A.dk, dv = A.dv, H = A.H;
    // two stages of a chunk's vectors (the next chunk's arrive while this one's tokens are walked), then what a chunk makes
    constexpr int NVEC = MODE == 1 ? 4 : (MODE == 2 ? 3 : 2);     // staged vectors of dk a token: k, q, then the removal rate (delta) and the decay (delta, gated linear attention)
    const size_t stage_floats = (size_t)NVEC * TC * KS + (size_t)TC * CTB + 2 * (size_t)TC;
    float* o_s = sm + 2 * stage_floats;            // [TC][CTB]
    float* m_s = o_s + TC * CTB;                   // [TC] memory: the running maximum after each token
    float* nqp = m_s + TC;                         // [TC][8] memory: n . q, one partial sum a warp
    float* a_s = nqp + TC * 8;                     // [TC] memory: what a token keeps of the state, exp(f + m_before - m_after)
    float* b_s = a_s + TC;                         // [TC] memory: what it adds, exp(i - m_after)
    float* tile = sm;                              // [dk][SPB], only before the first and after the last chunk

    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CTB;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = warp * CW + lane % CW, rg = lane / CW, r0 = rg * NR;
    const int t_begin = A.q_start[seq], t_end = A.q_start[seq + 1];
    if (t_begin >= t_end) return;
    const int slot = A.state_slot[seq];
    if (slot < 0 || slot >= A.num_slots) {
        if (tid == 0) report_status(A.status, SPY_STATUS_BAD_PAGE, t_begin);
        return;
    }
    float* st = A.state + ((size_t)slot * H + h) * A.record;
    for (int idx = tid; idx < dk * CTB; idx += THREADS) {
        const int r = idx / CTB, c = idx % CTB;
        tile[r * SPB + c] = c0 + c < dv ? st[(size_t)r * dv + c0 + c] : 0.f;
    }
    // n and m: a copy for every 8 columns of the state (the narrowest tile); a block reads the copy of its first 8 columns and
    // writes those of all its columns, so that every copy is the same whatever tiles the steps before and after use
    float* st_nm = st + (size_t)dk * dv + (size_t)(c0 / 8) * (dk + 1);
    const int copies = min(CTB / 8, (dv + 7) / 8 - c0 / 8);
    float m = 0.f, n_reg[4] = {0.f, 0.f, 0.f, 0.f};                           // n: the rows tid, tid + 256, ... (dk <= 1024)
    if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (tid + j * THREADS < dk) n_reg[j] = st_nm[tid + j * THREADS];
        m = st_nm[dk];
    }
    __syncthreads();
    float Sr[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) Sr[i] = r0 + i < dk ? tile[(r0 + i) * SPB + col] : 0.f;

    // whether a token's vectors start on 16-byte boundaries in the projection (and in the decay's pre-activation)
    const bool aligned = (dk & 3) == 0 && (A.ld & 3) == 0 && ((A.off_k | A.off_q) & 3) == 0 && (reinterpret_cast<uintptr_t>(A.proj) & 15) == 0 &&
                         (MODE == 0 || (((MODE == 1 ? A.off_x1 : 0) & 3) == 0 && (reinterpret_cast<uintptr_t>(A.extra) & 15) == 0));
    // Requests a chunk's vectors into a stage: 16-byte asynchronous copies where the columns allow it (all under way at once),
    // else plain loads; v and the gates' pre-activations by 4-byte copies.  What is made of them (the scaled q, the sigmoid of
    // the removal rate, the decay, the capped gates) is worked out in place once they have landed.
    auto request = [&](int t0, int stage) {
        const int n_tok = min(TC, t_end - t0);
        float* k_s = sm + stage * stage_floats;
        float* q_s = k_s + (size_t)TC * KS;
        float* x1_s = q_s + (size_t)TC * KS;
        float* x2_s = x1_s + (MODE == 1 ? (size_t)TC * KS : 0);
        float* v_s = x2_s + (MODE != 0 ? (size_t)TC * KS : 0);
        float* g1_s = v_s + TC * CTB;
        float* g2_s = g1_s + TC;
        if (aligned) {
            const int quads = dk >> 2;
            for (int idx = tid; idx < n_tok * quads; idx += THREADS) {
                const int tt = idx / quads, qd = idx - tt * quads, c = h * dk + 4 * qd;
                const float* row = A.proj + (size_t)(t0 + tt) * A.ld;
                cp_async16(k_s + tt * KS + 4 * qd, row + A.off_k + c);
                cp_async16(q_s + tt * KS + 4 * qd, row + A.off_q + c);
                if (MODE == 1) cp_async16(x1_s + tt * KS + 4 * qd, row + A.off_x1 + c);
                if (MODE != 0) cp_async16(x2_s + tt * KS + 4 * qd, A.extra + (size_t)(t0 + tt) * H * dk + c);
            }
        } else {
            for (int idx = tid; idx < n_tok * dk; idx += THREADS) {
                const int tt = idx / dk, r = idx - tt * dk, c = h * dk + r;
                const float* row = A.proj + (size_t)(t0 + tt) * A.ld;
                cp_async4(k_s + tt * KS + r, row + A.off_k + c);
                cp_async4(q_s + tt * KS + r, row + A.off_q + c);
                if (MODE == 1) cp_async4(x1_s + tt * KS + r, row + A.off_x1 + c);
                if (MODE != 0) cp_async4(x2_s + tt * KS + r, A.extra + (size_t)(t0 + tt) * H * dk + c);
            }
        }
        if (KS > dk) {
            const int pad = KS - dk;
            for (int idx = tid; idx < n_tok * pad; idx += THREADS) {
                const int tt = idx / pad, r = dk + idx - tt * pad;
                k_s[tt * KS + r] = 0.f;
                q_s[tt * KS + r] = 0.f;
                if (MODE == 1) x1_s[tt * KS + r] = 0.f;
                if (MODE != 0) x2_s[tt * KS + r] = 0.f;
            }
        }
        for (int idx = tid; idx < n_tok * CTB; idx += THREADS) {
            const int tt = idx / CTB, c = idx % CTB;
            if (c0 + c < dv) cp_async4(v_s + idx, A.proj + (size_t)(t0 + tt) * A.ld + A.off_v + h * dv + c0 + c);
            else v_s[idx] = 0.f;
        }
        if (MODE == 0 && tid < n_tok) {
            const float* row = A.proj + (size_t)(t0 + tid) * A.ld;
            cp_async4(g1_s + tid, row + A.off_x1 + h);
            cp_async4(g2_s + tid, row + A.off_x2 + h);
        }
    };
    __syncthreads();                               // the tile has been read: its place is the stages' now
    request(t_begin, 0);
    int stage = 0;
    for (int t0 = t_begin; t0 < t_end; t0 += TC, stage ^= 1) {
        const int n_tok = min(TC, t_end - t0);
        float* k_s = sm + stage * stage_floats;
        float* q_s = k_s + (size_t)TC * KS;
        float* x1_s = q_s + (size_t)TC * KS;
        float* x2_s = x1_s + (MODE == 1 ? (size_t)TC * KS : 0);
        float* v_s = x2_s + (MODE != 0 ? (size_t)TC * KS : 0);
        float* g1_s = v_s + TC * CTB;
        float* g2_s = g1_s + TC;
        cp_async_wait_all();
        __syncthreads();                           // this chunk's vectors have landed; the chunk before has been stored
        for (int idx = tid; idx < n_tok * dk; idx += THREADS) {
            const int tt = idx / dk, r = idx - tt * dk, c = h * dk + r;
            if (MODE == 0) {
                q_s[tt * KS + r] *= A.q_scale;
            } else if (MODE == 2) {
                q_s[tt * KS + r] *= A.q_scale;
                x2_s[tt * KS + r] = expf(log_sigmoidf_(x2_s[tt * KS + r] + A.bias2[c]) * A.cap);
            } else {
                x1_s[tt * KS + r] = sigmoidf_(x1_s[tt * KS + r] + A.bias1[c]);
                x2_s[tt * KS + r] = expf(-0.60653065971263342f * sigmoidf_(x2_s[tt * KS + r] + A.bias2[c]));   // exp(-1/2) = 0.6065...
            }
        }
        if (MODE == 0 && tid < n_tok) {
            g1_s[tid] = A.cap * tanhf((g1_s[tid] + A.bias1[h]) / A.cap);
            g2_s[tid] = log_sigmoidf_(A.cap * tanhf((g2_s[tid] + A.bias2[h]) / A.cap));
        }
        __syncthreads();
        if (MODE == 1) {
            for (int tt = warp; tt < n_tok; tt += THREADS / 32) {
                float ksq = 0.f;
                for (int r = lane; r < dk; r += 32) ksq += k_s[tt * KS + r] * k_s[tt * KS + r];
                ksq = warp_sum(ksq);
                if (lane == 0) g1_s[tt] = 1.0f / sqrtf(ksq + 1e-6f);
            }
            __syncthreads();
        }
        if (MODE == 0) {
            // The running maximum is a chain through the chunk's tokens (an addition and a maximum each), walked by one
            // lane; the two exponentials of every token, which need only the maxima before and after it, are then worked
            // out by a lane each.  The numbers are those of a token-by-token walk.
            if (warp == 0) {         // a chunk has at most 32 tokens: lane tt keeps token tt's gates, the chain runs through shuffles
                const float ig = lane < n_tok ? g1_s[lane] : 0.f, fg = lane < n_tok ? g2_s[lane] : 0.f;
                float mm = m, before = m, after = m;
                for (int tt = 0; tt < n_tok; ++tt) {
                    const float f_t = __shfl_sync(0xffffffffu, fg, tt), i_t = __shfl_sync(0xffffffffu, ig, tt);
                    const float next = fmaxf(f_t + mm, i_t);
                    if (lane == tt) {
                        before = mm;
                        after = next;
                    }
                    mm = next;
                }
                if (lane < n_tok) {
                    m_s[lane] = after;
                    a_s[lane] = expf(fg + before - after);
                    b_s[lane] = expf(ig - after);
                }
            }
            __syncthreads();
            m = m_s[n_tok - 1];
        }
        if (t0 + TC < t_end) request(t0 + TC, stage ^ 1);     // the stage that the chunk before used; every thread is past that chunk
        constexpr int U = NR <= 8 ? 8 : 4;         // tokens walked at a time (their reductions run together); fewer when a thread's rows take many registers
        for (int tt0 = 0; tt0 < n_tok; tt0 += U) {
            float acc[U], nq[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int tt = tt0 + u;
                acc[u] = 0.f;
                nq[u] = 0.f;
                if (tt >= n_tok) continue;         // the same for every thread
                const float* __restrict__ k = k_s + tt * KS + r0;
                const float* __restrict__ q = q_s + tt * KS + r0;
                const float v_c = v_s[tt * CTB + col];
                if (MODE == 0) {
                    const float a_t = a_s[tt], b_t = b_s[tt];
                    float part[4] = {0.f, 0.f, 0.f, 0.f};     // several short chains of sums instead of one long one
#pragma unroll
                    for (int i0 = 0; i0 < NR; i0 += V4) {
                        float kk[V4], qq[V4];
                        if (V4 == 4) {
                            *reinterpret_cast<float4*>(kk) = *reinterpret_cast<const float4*>(k + i0);
                            *reinterpret_cast<float4*>(qq) = *reinterpret_cast<const float4*>(q + i0);
                        } else {
#pragma unroll
                            for (int e = 0; e < V4; ++e) { kk[e] = k[i0 + e]; qq[e] = q[i0 + e]; }
                        }
#pragma unroll
                        for (int e = 0; e < V4; ++e) {
                            const float s = a_t * Sr[i0 + e] + (b_t * kk[e]) * v_c;
                            Sr[i0 + e] = s;
                            part[e & 3] = fmaf(s, qq[e], part[e & 3]);
                        }
                    }
                    acc[u] = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = tid + j * THREADS;
                        if (r < dk) {
                            n_reg[j] = a_t * n_reg[j] + b_t * k_s[tt * KS + r];
                            nq[u] += n_reg[j] * q_s[tt * KS + r];
                        }
                    }
                } else if (MODE == 2) {
                    const float* __restrict__ decay = x2_s + tt * KS + r0;
                    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i0 = 0; i0 < NR; i0 += V4) {
                        float kk[V4], qq[V4], dd[V4];
                        if (V4 == 4) {
                            *reinterpret_cast<float4*>(kk) = *reinterpret_cast<const float4*>(k + i0);
                            *reinterpret_cast<float4*>(qq) = *reinterpret_cast<const float4*>(q + i0);
                            *reinterpret_cast<float4*>(dd) = *reinterpret_cast<const float4*>(decay + i0);
                        } else {
#pragma unroll
                            for (int e = 0; e < V4; ++e) { kk[e] = k[i0 + e]; qq[e] = q[i0 + e]; dd[e] = decay[i0 + e]; }
                        }
#pragma unroll
                        for (int e = 0; e < V4; ++e) {
                            const float s = fmaf(dd[e], Sr[i0 + e], kk[e] * v_c);
                            Sr[i0 + e] = s;
                            part[e & 3] = fmaf(s, qq[e], part[e & 3]);
                        }
                    }
                    acc[u] = (part[0] + part[1]) + (part[2] + part[3]);
                } else {
                    const float inv = g1_s[tt];
                    const float* __restrict__ rate = x1_s + tt * KS + r0;
                    const float* __restrict__ decay = x2_s + tt * KS + r0;
                    float part[4] = {0.f, 0.f, 0.f, 0.f};     // several short chains of sums instead of one long one
#pragma unroll
                    for (int i = 0; i < NR; ++i) part[i & 3] = fmaf(k[i] * inv, Sr[i], part[i & 3]);
                    float us = (part[0] + part[1]) + (part[2] + part[3]);
                    part[0] = part[1] = part[2] = part[3] = 0.f;
#pragma unroll
                    for (int o = CW; o <= 16; o <<= 1) us += __shfl_xor_sync(0xffffffffu, us, o);
#pragma unroll
                    for (int i0 = 0; i0 < NR; i0 += V4) {
                        float kk[V4], qq[V4], rr[V4], dd[V4];
                        if (V4 == 4) {
                            *reinterpret_cast<float4*>(kk) = *reinterpret_cast<const float4*>(k + i0);
                            *reinterpret_cast<float4*>(qq) = *reinterpret_cast<const float4*>(q + i0);
                            *reinterpret_cast<float4*>(rr) = *reinterpret_cast<const float4*>(rate + i0);
                            *reinterpret_cast<float4*>(dd) = *reinterpret_cast<const float4*>(decay + i0);
                        } else {
#pragma unroll
                            for (int e = 0; e < V4; ++e) { kk[e] = k[i0 + e]; qq[e] = q[i0 + e]; rr[e] = rate[i0 + e]; dd[e] = decay[i0 + e]; }
                        }
#pragma unroll
                        for (int e = 0; e < V4; ++e) {
                            const float u_r = kk[e] * inv;
                            const float s = dd[e] * Sr[i0 + e] - (rr[e] * u_r) * us + kk[e] * v_c;
                            Sr[i0 + e] = s;
                            part[e & 3] = fmaf(s, qq[e], part[e & 3]);
                        }
                    }
                    acc[u] = (part[0] + part[1]) + (part[2] + part[3]);
                }
            }
#pragma unroll
            for (int o = CW; o <= 16; o <<= 1) {
#pragma unroll
                for (int u = 0; u < U; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
            }
            if (MODE == 0) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int u = 0; u < U; ++u) nq[u] += __shfl_xor_sync(0xffffffffu, nq[u], o);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (tt0 + u < n_tok) {
                    if (rg == 0) o_s[(tt0 + u) * CTB + col] = acc[u];
                    if (MODE == 0 && lane == 0) nqp[(tt0 + u) * 8 + warp] = nq[u];
                }
            }
        }
        __syncthreads();
        for (int idx = tid; idx < n_tok * CTB; idx += THREADS) {
            const int tt = idx / CTB, c = idx % CTB;
            if (c0 + c >= dv) continue;
            float o = o_s[idx];
            if (MODE == 0) {
                float nq = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) nq += nqp[tt * 8 + w];
                o = o / (fmaxf(fabsf(nq), expf(-m_s[tt])) + 1e-6f);
            }
            A.out[(size_t)(t0 + tt) * H * dv + h * dv + c0 + c] = o;
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NR; ++i)
        if (r0 + i < dk) tile[(r0 + i) * SPB + col] = Sr[i];
    __syncthreads();
    for (int idx = tid; idx < dk * CTB; idx += THREADS) {
        const int r = idx / CTB, c = idx % CTB;
        if (c0 + c < dv) st[(size_t)r * dv + c0 + c] = tile[r * SPB + c];
    }
    if (MODE == 0) {
        for (int cp = 0; cp < copies; ++cp) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (tid + j * THREADS < dk) st_nm[(size_t)cp * (dk + 1) + tid + j * THREADS] = n_reg[j];
            if (tid == 0) st_nm[(size_t)cp * (dk + 1) + dk] = m;
        }
    }
    pdl_launch_dependents();
}

// Decoding (every request brings one token): the state's way through memory is all there is to do, so the kernel is built
// to keep much of it under way: a lane owns a column of the tile (a warp reads and writes whole 128-byte rows), a warp owns
// NR consecutive rows, the loads of a thread's rows are issued before anything else, and several blocks share an SM.  Sums
// over the rows cross the warps through shared memory.
template <int MODE, int NR>
__global__ void __launch_bounds__(THREADS, NR <= 16 ? 4 : 1) scan_decode_kernel(ScanArgs A)
{
    __shared__ float red[8][CT], red2[8][CT], part[8], nqp[8];
    extern __shared__ __align__(16) float vec[];      // k, q and, for the delta rule, the removal rate and the decay: dk each
    pdl_enter();
    const int dk = A.dk, dv = A.dv, H = A.H;
    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CT;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, r0 = warp * NR;
    const int t = A.q_start[seq];
    if (A.q_start[seq + 1] <= t) return;
    const int slot = A.state_slot[seq];
    if (slot < 0 || slot >= A.num_slots) {
        if (tid == 0) report_status(A.status, SPY_STATUS_BAD_PAGE, t);
        return;
    }
    const bool col_ok = c0 + lane < dv;
    float* st = A.state + ((size_t)slot * H + h) * A.record;
    float Sr[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) Sr[i] = (r0 + i < dk && col_ok) ? st[(size_t)(r0 + i) * dv + c0 + lane] : 0.f;
    const float* row = A.proj + (size_t)t * A.ld;
    float *k_s = vec, *q_s = vec + dk, *x1_s = vec + 2 * dk, *x2_s = vec + (MODE == 1 ? 3 : 2) * dk;     // gated linear attention has no x1
    float a = 1.f, b = 0.f, m_new = 0.f, ksq = 0.f, nq = 0.f;
    float* st_nm = st + (size_t)dk * dv + (size_t)(c0 / 8) * (dk + 1);      // n and m: a copy for every 8 columns; the first of this tile's is read, all of them are written
    const int copies = min(CT / 8, (dv + 7) / 8 - c0 / 8);
    if (MODE == 0) {
        const float ig = A.cap * tanhf((row[A.off_x1 + h] + A.bias1[h]) / A.cap);
        const float fg = log_sigmoidf_(A.cap * tanhf((row[A.off_x2 + h] + A.bias2[h]) / A.cap));
        const float m = st_nm[dk];
        m_new = fmaxf(fg + m, ig);
        a = expf(fg + m - m_new);
        b = expf(ig - m_new);
    }
    for (int r = tid; r < dk; r += THREADS) {
        const int c = h * dk + r;
        const float kr = row[A.off_k + c], qr = row[A.off_q + c] * A.q_scale;
        k_s[r] = kr;
        q_s[r] = qr;
        if (MODE == 0) {
            const float n = a * st_nm[r] + b * kr;
            for (int cp = 0; cp < copies; ++cp) st_nm[(size_t)cp * (dk + 1) + r] = n;
            nq += n * qr;
        } else if (MODE == 2) {
            x2_s[r] = expf(log_sigmoidf_(A.extra[(size_t)t * H * dk + c] + A.bias2[c]) * A.cap);
        } else {
            x1_s[r] = sigmoidf_(row[A.off_x1 + c] + A.bias1[c]);
            x2_s[r] = expf(-0.60653065971263342f * sigmoidf_(A.extra[(size_t)t * H * dk + c] + A.bias2[c]));
            ksq += kr * kr;
        }
    }
    if (MODE == 0) {
        nq = warp_sum(nq);
        if (lane == 0) nqp[warp] = nq;
    } else if (MODE == 1) {
        ksq = warp_sum(ksq);
        if (lane == 0) part[warp] = ksq;
    }
    __syncthreads();
    const float v_c = col_ok ? row[A.off_v + h * dv + c0 + lane] : 0.f;
    float acc = 0.f;
    if (MODE == 0) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = r0 + i;
            if (r < dk) {
                const float s = a * Sr[i] + (b * k_s[r]) * v_c;
                if (col_ok) st[(size_t)r * dv + c0 + lane] = s;
                acc = fmaf(s, q_s[r], acc);
            }
        }
        red[warp][lane] = acc;
        __syncthreads();
        if (warp == 0 && col_ok) {
            float o = 0.f, n = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) { o += red[w][lane]; n += nqp[w]; }
            A.out[(size_t)t * H * dv + h * dv + c0 + lane] = o / (fmaxf(fabsf(n), expf(-m_new)) + 1e-6f);
        }
        if (tid == 0)
            for (int cp = 0; cp < copies; ++cp) st_nm[(size_t)cp * (dk + 1) + dk] = m_new;
    } else if (MODE == 2) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = r0 + i;
            if (r < dk) {
                const float s = fmaf(x2_s[r], Sr[i], k_s[r] * v_c);
                if (col_ok) st[(size_t)r * dv + c0 + lane] = s;
                acc = fmaf(s, q_s[r], acc);
            }
        }
        red2[warp][lane] = acc;
        __syncthreads();
        if (warp == 0 && col_ok) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) o += red2[w][lane];
            A.out[(size_t)t * H * dv + h * dv + c0 + lane] = o;
        }
    } else {
        float sq = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) sq += part[w];
        const float inv = 1.0f / sqrtf(sq + 1e-6f);
        float us = 0.f;
#pragma unroll
        for (int i = 0; i < NR; ++i)
            if (r0 + i < dk) us = fmaf(k_s[r0 + i] * inv, Sr[i], us);
        red[warp][lane] = us;
        __syncthreads();
        us = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) us += red[w][lane];
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = r0 + i;
            if (r < dk) {
                const float u = k_s[r] * inv;
                const float s = x2_s[r] * Sr[i] - (x1_s[r] * u) * us + k_s[r] * v_c;
                if (col_ok) st[(size_t)r * dv + c0 + lane] = s;
                acc = fmaf(s, q_s[r], acc);
            }
        }
        red2[warp][lane] = acc;
        __syncthreads();
        if (warp == 0 && col_ok) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) o += red2[w][lane];
            A.out[(size_t)t * H * dv + h * dv + c0 + lane] = o;
        }
    }
}

template <int MODE, int RG> static int launch_scan_rg(ScanArgs& A, int num_seqs, int longest, cudaStream_t stream)
{
    constexpr int CTB = 8 * (32 / RG);
    const int tiles = (A.dv + CTB - 1) / CTB;
    int nr = 2;
    while (RG * nr < A.dk) nr *= 2;
    if (nr > 64) SPY_FAIL("recurrence: a key size of %d exceeds the kernel's %d", A.dk, 64 * RG);
    // tokens a chunk: 32, fewer when a request never brings that many or when the vectors of 32 would not fit
    int tc = 32;
    while (tc > 1 && tc / 2 >= longest) tc /= 2;
    auto bytes = [&](int n) {
        const size_t stage = (MODE == 1 ? 4 : (MODE == 2 ? 3 : 2)) * (size_t)n * RG * nr + (size_t)n * CTB + 2 * (size_t)n;      // one stage of a chunk's vectors
        const size_t staged = (2 * stage + (size_t)n * CTB + 11 * (size_t)n) * sizeof(float);
        const size_t tile = (size_t)A.dk * (CTB + 4) * sizeof(float);
        return staged > tile ? staged : tile;
    };
    while (tc > 1 && bytes(tc) > 100 * 1024) tc /= 2;
    const size_t smem = bytes(tc);
    if (smem > 227 * 1024) SPY_FAIL("recurrence: a key size of %d does not fit a block's shared memory", A.dk);
    void (*kernel)(ScanArgs, int) = nullptr;
    switch (nr) {
        case 2: kernel = scan_kernel<MODE, 2, RG>; break;
        case 4: kernel = scan_kernel<MODE, 4, RG>; break;
        case 8: kernel = scan_kernel<MODE, 8, RG>; break;
        case 16: kernel = scan_kernel<MODE, 16, RG>; break;
        case 32: kernel = scan_kernel<MODE, 32, RG>; break;
        default: kernel = scan_kernel<MODE, 64, RG>; break;
    }
    if (smem > 48 * 1024) SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    spy_launch_in_order(kernel, dim3(num_seqs, A.H, tiles), dim3(THREADS), smem, stream, A, tc);
    SPY_CHECK_LAUNCH("recurrence scan");
    return 0;
}

template <int MODE> static int launch_scan_mode(ScanArgs& A, int num_seqs, int longest, cudaStream_t stream)
{
    if (longest <= 1) {     // every request brings one token
        const int tiles = (A.dv + CT - 1) / CT;
        int nr = 2;
        while (8 * nr < A.dk) nr *= 2;
        if (nr > 64) SPY_FAIL("recurrence: a key size of %d exceeds the kernel's 512", A.dk);
        void (*dk_kernel)(ScanArgs) = nullptr;
        switch (nr) {
            case 2: dk_kernel = scan_decode_kernel<MODE, 2>; break;
            case 4: dk_kernel = scan_decode_kernel<MODE, 4>; break;
            case 8: dk_kernel = scan_decode_kernel<MODE, 8>; break;
            case 16: dk_kernel = scan_decode_kernel<MODE, 16>; break;
            case 32: dk_kernel = scan_decode_kernel<MODE, 32>; break;
            default: dk_kernel = scan_decode_kernel<MODE, 64>; break;
        }
        const size_t vec_bytes = (MODE == 1 ? 4 : (MODE == 2 ? 3 : 2)) * (size_t)A.dk * sizeof(float);
        spy_launch(dk_kernel, dim3(num_seqs, A.H, tiles), dim3(THREADS), vec_bytes, stream, A);
        SPY_CHECK_LAUNCH("recurrence scan (decoding)");
        return 0;
    }
    // the widest tiles (32, 16 or 8 columns a block) that still give (nearly) every SM a block; key sizes above 512 need the narrower ones
    const int sms = spy_sm_count();
    const long long heads = (long long)num_seqs * A.H;
    static int forced = -1;                      // SPYINFER_SCAN_RG = 8, 16 or 32 in the environment fixes the tile width (for measurements)
    if (forced < 0) {
        const char* e = getenv("SPYINFER_SCAN_RG");
        forced = e != nullptr ? atoi(e) : 0;
    }
    if (forced == 8 && A.dk <= 512) return launch_scan_rg<MODE, 8>(A, num_seqs, longest, stream);
    if (forced == 16 && A.dk <= 1024) return launch_scan_rg<MODE, 16>(A, num_seqs, longest, stream);
    if (forced == 32) return launch_scan_rg<MODE, 32>(A, num_seqs, longest, stream);
    // measured on one request of 8 heads, 128 x 256: 64 blocks of 32 columns 0.79 ms, 128 of 16 columns 0.64, 256 of 8 columns 0.75
    if (A.dk <= 512 && heads * ((A.dv + 31) / 32) >= sms) return launch_scan_rg<MODE, 8>(A, num_seqs, longest, stream);
    if (A.dk <= 1024 && 4 * heads * ((A.dv + 15) / 16) >= 3 * sms) return launch_scan_rg<MODE, 16>(A, num_seqs, longest, stream);
    return launch_scan_rg<MODE, 32>(A, num_seqs, longest, stream);
}

static int launch_scan(int mode, ScanArgs& A, int num_seqs, int longest, cudaStream_t stream)
{
    if (num_seqs <= 0) return 0;
    if (A.H <= 0 || A.dk <= 0 || A.dv <= 0) SPY_FAIL("recurrence: heads %d, key size %d and value size %d must be positive", A.H, A.dk, A.dv);
    if (A.H > 65535) SPY_FAIL("recurrence: %d heads exceed the grid limit", A.H);
    if ((A.dv + CT - 1) / CT > 65535) SPY_FAIL("recurrence: a value size of %d exceeds the grid limit", A.dv);
    if (mode == 2) return launch_scan_mode<2>(A, num_seqs, longest, stream);
    return mode == 0 ? launch_scan_mode<0>(A, num_seqs, longest, stream) : launch_scan_mode<1>(A, num_seqs, longest, stream);
}

// State record of one head, in floats.
extern "C" long long spy_mlstm_record(int dk, int dv) { return ((long long)dk * dv + (long long)((dv + 7) / 8) * (dk + 1) + 3) / 4 * 4; }

extern "C" int spy_mlstm_scan(const float* proj, long long ld, int off_q, int off_k, int off_v, int off_i, int off_f, const float* bias_i, const float* bias_f,
                              float* state, int num_slots, const int* q_start, const int* state_slot, int num_seqs, int longest, float* out, int H, int dk,
                              int dv, float q_scale, float cap, int* status, cudaStream_t stream)
{
    if (!(cap > 0.f)) SPY_FAIL("mlstm: the gates' cap must be positive");
    ScanArgs A = {proj, ld, off_q, off_k, off_v, off_i, off_f, nullptr, bias_i, bias_f, state, spy_mlstm_record(dk, dv), num_slots, q_start, state_slot, out,
                  H, dk, dv, q_scale, cap, status};
    return launch_scan(0, A, num_seqs, longest, stream);
}

extern "C" int spy_delta_scan(const float* proj, long long ld, int off_r, int off_k, int off_v, int off_a, const float* decay_pre, const float* bias_a,
                              const float* decay_offset, float* state, int num_slots, const int* q_start, const int* state_slot, int num_seqs, int longest,
                              float* out, int H, int dk, int* status, cudaStream_t stream)
{
    ScanArgs A = {proj, ld, off_r, off_k, off_v, off_a, 0, decay_pre, bias_a, decay_offset, state, (long long)dk * dk, num_slots, q_start, state_slot, out,
                  H, dk, dk, 1.0f, 1.0f, status};
    return launch_scan(1, A, num_seqs, longest, stream);
}

// Gated linear attention with a decay per key channel: proj holds q, k, v at `off_*`; decay_pre [T, H * dk] the decay's
// pre-activation z, to which decay_bias [H * dk] is added: a = exp(logsigmoid(z + bias) / tau).  q is scaled by q_scale.
extern "C" int spy_gla_scan(const float* proj, long long ld, int off_q, int off_k, int off_v, const float* decay_pre, const float* decay_bias, float inv_tau,
                            float* state, int num_slots, const int* q_start, const int* state_slot, int num_seqs, int longest, float* out, int H, int dk, int dv,
                            float q_scale, int* status, cudaStream_t stream)
{
    if (!(inv_tau > 0.f)) SPY_FAIL("gated linear attention: tau must be positive");
    ScanArgs A = {proj, ld, off_q, off_k, off_v, 0, 0, decay_pre, nullptr, decay_bias, state, (long long)dk * dv, num_slots, q_start, state_slot, out,
                  H, dk, dv, q_scale, inv_tau, status};
    return launch_scan(2, A, num_seqs, longest, stream);
}

// ---- what follows a recurrence: unit root mean square per head, a weight, a gate (sigmoid, or SiLU) -------------
// One warp a (token, head) row, eight rows a block: the row's sum of squares is a sum inside the warp.
template <typename TO>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ proj, long long ld, int off_g, const float* __restrict__ weight,
                                       TO* __restrict__ out, long long rows, int H, int dv, float eps, int gate_act)
{
    pdl_enter();
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = row / H;
    const int h = (int)(row - t * H);
    const float* src = o + row * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* g = proj + t * ld + off_g + h * dv;
    for (int c = lane; c < dv; c += 32) {
        const float gate = gate_act == 1 ? g[c] * sigmoidf_(g[c]) : sigmoidf_(g[c]);
        out[row * dv + c] = from_f32<TO>(((src[c] * inv) * weight[h * dv + c]) * gate);
    }
}

extern "C" int spy_gated_head_norm(const float* o, const float* proj, long long ld, int off_g, const float* weight, void* out, int out_dtype, int tokens,
                                   int H, int dv, float eps, cudaStream_t stream, int gate_act)
{
    if (gate_act != 0 && gate_act != 1) SPY_FAIL("gated_head_norm: gate activation %d (0: sigmoid, 1: SiLU)", gate_act);
    if (tokens <= 0) return 0;
    if (H <= 0 || dv <= 0) SPY_FAIL("gated_head_norm: %d heads of %d", H, dv);
    const long long rows = (long long)tokens * H, blocks = (rows + 7) / 8;
    if (blocks > 0x7fffffffLL) SPY_FAIL("gated_head_norm: %lld rows exceed the grid limit", rows);
    SPY_DISPATCH_DTYPE(out_dtype, TO, {
        spy_launch(gated_head_norm_kernel<TO>, dim3((unsigned)blocks), dim3(256), 0, stream, o, proj, ld, off_g, weight, (TO*)out, rows, H, dv, eps, gate_act);
    })
    SPY_CHECK_LAUNCH("gated_head_norm");
    return 0;
}

// out[t, j] = act(proj[t, off + j]) for j < n: the inner activation of a two-step (low-rank) projection; act 0: tanh, 1: none.
template <typename TO>
__global__ void tanh_cols_kernel(const float* __restrict__ proj, long long ld, int off, int n, TO* __restrict__ out, long long total, int act)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long t = i / n;
        const float x = proj[t * ld + off + (i - t * n)];
        out[i] = from_f32<TO>(act == 0 ? tanhf(x) : x);
    }
}

extern "C" int spy_tanh_cols(const float* proj, long long ld, int off, int n, void* out, int out_dtype, int tokens, cudaStream_t stream, int act)
{
    if (tokens <= 0 || n <= 0) return 0;
    if (act != 0 && act != 1) SPY_FAIL("tanh_cols: activation %d (0: tanh, 1: none)", act);
    const long long total = (long long)tokens * n;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(out_dtype, TO, {
        spy_launch(tanh_cols_kernel<TO>, dim3((int)blocks), dim3(256), 0, stream, proj, ld, off, n, (TO*)out, total, act);
    })
    SPY_CHECK_LAUNCH("tanh_cols");
    return 0;
}
