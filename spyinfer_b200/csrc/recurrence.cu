// Linear recurrences over a matrix state per (request, head), carried from token to token in 32-bit:
//   * the gated matrix memory (mLSTM):       S = a S + b k v^T,  n = a n + b k,  o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
//                                            with log gates i, f, the running maximum m' = max(f + m, i) (m starts at 0),
//                                            a = exp(f + m - m'), b = exp(i - m');
//   * the generalised delta rule:            S = diag(w) S - (r u)(u^T S) + k v^T,  o = S^T q,  u = k / sqrt(sum k^2 + 1e-6),
//                                            both terms reading the old S, w a decay and r a removal rate per key channel;
// and what follows both: each head's output divided by its root mean square, times a weight, times a sigmoid gate.
//
// One kernel serves prompt portions and decoding: a block owns CT = 32 value columns of one (request, head), holds its
// [dk x 32] tile of S in shared memory and walks the request's tokens of this step in order (`longest`: the most tokens a
// request of the step brings, or more; it only sizes the chunks that are staged in shared memory).  The columns of S do not
// depend on one another, so the tiles of a head run side by side; the vector n and the maximum m, which all tiles of a head
// need, are kept and updated by each tile for itself (dk + 1 numbers a tile in the state record: no tile ever reads what
// another writes, whenever their blocks happen to run).  The per-token arithmetic is the same
// whatever the step's cut, so a position's result does not depend on how its request was cut into steps.
//
// Inputs are columns of one 32-bit activation matrix `proj` [T, ld] (the fused projection of the mixer's input).
#include "common.cuh"

SPY_MODULE(spy_recurrence)

constexpr int CT = 32;   // value columns a block owns

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float log_sigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct ScanArgs {
    const float* proj;      // [T, ld]
    long long ld;
    int off_q, off_k, off_v, off_x1, off_x2;   // columns of q (or r), k, v; mLSTM: i and f pre-activations; delta: the removal rate's pre-activation (x2 unused)
    const float* extra;     // delta: the decay's pre-activation [T, H * dk]
    const float* bias1;     // mLSTM: bias of i [H];   delta: bias of the removal rate [H * dk]
    const float* bias2;     // mLSTM: bias of f [H];   delta: the decay's offset [H * dk]
    float* state;           // [slots, H, record]
    long long record;       // floats a head: mLSTM dk * dv + (dk + 1) a column tile (padded to 4); delta dk * dv
    int num_slots;
    const int* q_start;     // [S + 1]
    const int* state_slot;  // [S]
    float* out;             // [T, H * dv]
    int H, dk, dv;
    float q_scale, cap;
    int* status;
};

constexpr int SP = CT + 4;        // floats between the rows of a state tile while it passes through shared memory
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
// token run beside those of the others and beside the next token's rows (nothing in S waits for them).  LIGHT: built
// for four blocks an SM (at most 64 registers), for decoding, where a block's time is the state's way through memory.
template <int MODE, int NR, bool LIGHT>   // MODE 0: gated matrix memory, 1: delta rule
__global__ void __launch_bounds__(THREADS, LIGHT ? 4 : 1) scan_kernel(ScanArgs A, int TC)
{
    extern __shared__ __align__(16) float sm[];
    pdl_enter();
    constexpr int KS = 8 * NR;                     // floats a staged vector takes
    constexpr int V4 = NR >= 4 ? 4 : NR;           // elements a load of a thread's rows brings
    const int dk = A.dk, dv = A.dv, H = A.H;
    float* k_s = sm;                               // [TC][KS]
    float* q_s = k_s + (size_t)TC * KS;            // [TC][KS]
    float* x1_s = q_s + (size_t)TC * KS;           // delta: removal rate [TC][KS]
    float* x2_s = x1_s + (MODE == 1 ? (size_t)TC * KS : 0);   // delta: decay [TC][KS]
    float* v_s = x2_s + (MODE == 1 ? (size_t)TC * KS : 0);    // [TC][CT]
    float* o_s = v_s + TC * CT;                    // [TC][CT]
    float* g1_s = o_s + TC * CT;                   // [TC] memory: log input gate; delta: 1 / |k|
    float* g2_s = g1_s + TC;                       // [TC] memory: log forget gate
    float* m_s = g2_s + TC;                        // [TC] memory: the running maximum after each token
    float* nqp = m_s + TC;                         // [TC][8] memory: n . q, one partial sum a warp
    float* tile = sm;                              // [dk][SP], only before the first and after the last chunk

    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CT;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = warp * 4 + (lane & 3), rg = lane >> 2, r0 = rg * NR;
    const int t_begin = A.q_start[seq], t_end = A.q_start[seq + 1];
    if (t_begin >= t_end) return;
    const int slot = A.state_slot[seq];
    if (slot < 0 || slot >= A.num_slots) {
        if (tid == 0) report_status(A.status, SPY_STATUS_BAD_PAGE, t_begin);
        return;
    }
    float* st = A.state + ((size_t)slot * H + h) * A.record;
    for (int idx = tid; idx < dk * CT; idx += THREADS) {
        const int r = idx / CT, c = idx % CT;
        tile[r * SP + c] = c0 + c < dv ? st[(size_t)r * dv + c0 + c] : 0.f;
    }
    float* st_nm = st + (size_t)dk * dv + (size_t)blockIdx.z * (dk + 1);      // this tile's own copy of n and m
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
    for (int i = 0; i < NR; ++i) Sr[i] = r0 + i < dk ? tile[(r0 + i) * SP + col] : 0.f;

    for (int t0 = t_begin; t0 < t_end; t0 += TC) {
        const int n_tok = min(TC, t_end - t0);
        __syncthreads();                           // the chunk before has been stored (the first time: the tile has been read)
        for (int idx = tid; idx < n_tok * KS; idx += THREADS) {
            const int tt = idx / KS, r = idx - tt * KS, c = h * dk + r;
            const float* row = A.proj + (size_t)(t0 + tt) * A.ld;
            const bool ok = r < dk;
            k_s[idx] = ok ? row[A.off_k + c] : 0.f;
            q_s[idx] = ok ? row[A.off_q + c] * A.q_scale : 0.f;
            if (MODE == 1) {
                x1_s[idx] = ok ? sigmoidf_(row[A.off_x1 + c] + A.bias1[c]) : 0.f;
                x2_s[idx] = ok ? expf(-0.60653065971263342f * sigmoidf_(A.extra[(size_t)(t0 + tt) * H * dk + c] + A.bias2[c])) : 0.f;   // exp(-1/2) = 0.6065...
            }
        }
        for (int idx = tid; idx < n_tok * CT; idx += THREADS) {
            const int tt = idx / CT, c = idx % CT;
            v_s[idx] = c0 + c < dv ? A.proj[(size_t)(t0 + tt) * A.ld + A.off_v + h * dv + c0 + c] : 0.f;
        }
        if (MODE == 0 && tid < n_tok) {
            const float* row = A.proj + (size_t)(t0 + tid) * A.ld;
            g1_s[tid] = A.cap * tanhf((row[A.off_x1 + h] + A.bias1[h]) / A.cap);
            g2_s[tid] = log_sigmoidf_(A.cap * tanhf((row[A.off_x2 + h] + A.bias2[h]) / A.cap));
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
        // the gates of the chunk's first token; those of the token after are worked out while a token's rows are
        float a = 1.f, b = 0.f, m_after = m;
        if (MODE == 0) {
            m_after = fmaxf(g2_s[0] + m, g1_s[0]);
            a = expf(g2_s[0] + m - m_after);
            b = expf(g1_s[0] - m_after);
        }
        constexpr int U = 4;
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
                const float v_c = v_s[tt * CT + col];
                if (MODE == 0) {
                    const float a_t = a, b_t = b;
                    m = m_after;
                    if (tt + 1 < n_tok) {
                        m_after = fmaxf(g2_s[tt + 1] + m, g1_s[tt + 1]);
                        a = expf(g2_s[tt + 1] + m - m_after);
                        b = expf(g1_s[tt + 1] - m_after);
                    }
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
                            acc[u] = fmaf(s, qq[e], acc[u]);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = tid + j * THREADS;
                        if (r < dk) {
                            n_reg[j] = a_t * n_reg[j] + b_t * k_s[tt * KS + r];
                            nq[u] += n_reg[j] * q_s[tt * KS + r];
                        }
                    }
                    if (tid == 0) m_s[tt] = m;
                } else {
                    const float inv = g1_s[tt];
                    const float* __restrict__ rate = x1_s + tt * KS + r0;
                    const float* __restrict__ decay = x2_s + tt * KS + r0;
                    float us = 0.f;
#pragma unroll
                    for (int i = 0; i < NR; ++i) us = fmaf(k[i] * inv, Sr[i], us);
                    us += __shfl_xor_sync(0xffffffffu, us, 4);
                    us += __shfl_xor_sync(0xffffffffu, us, 8);
                    us += __shfl_xor_sync(0xffffffffu, us, 16);
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
                            acc[u] = fmaf(s, qq[e], acc[u]);
                        }
                    }
                }
            }
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
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
                    if (rg == 0) o_s[(tt0 + u) * CT + col] = acc[u];
                    if (MODE == 0 && lane == 0) nqp[(tt0 + u) * 8 + warp] = nq[u];
                }
            }
        }
        __syncthreads();
        for (int idx = tid; idx < n_tok * CT; idx += THREADS) {
            const int tt = idx / CT, c = idx % CT;
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
        if (r0 + i < dk) tile[(r0 + i) * SP + col] = Sr[i];
    __syncthreads();
    for (int idx = tid; idx < dk * CT; idx += THREADS) {
        const int r = idx / CT, c = idx % CT;
        if (c0 + c < dv) st[(size_t)r * dv + c0 + c] = tile[r * SP + c];
    }
    if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (tid + j * THREADS < dk) st_nm[tid + j * THREADS] = n_reg[j];
        if (tid == 0) st_nm[dk] = m;
    }
}

template <int MODE> static int launch_scan_mode(ScanArgs& A, int num_seqs, int longest, cudaStream_t stream)
{
    const int tiles = (A.dv + CT - 1) / CT;
    int nr = 2;
    while (8 * nr < A.dk) nr *= 2;
    if (nr > 64) SPY_FAIL("recurrence: a key size of %d exceeds the kernel's 512", A.dk);
    // tokens a chunk: 32, fewer when a request never brings that many (decoding) or when the vectors of 32 would not fit
    int tc = 32;
    while (tc > 1 && tc / 2 >= longest) tc /= 2;
    auto bytes = [&](int n) {
        const size_t staged = ((MODE == 1 ? 4 : 2) * (size_t)n * 8 * nr + 2 * (size_t)n * CT + 11 * (size_t)n) * sizeof(float);
        const size_t tile = (size_t)A.dk * SP * sizeof(float);
        return staged > tile ? staged : tile;
    };
    while (tc > 1 && bytes(tc) > 64 * 1024) tc /= 2;
    const size_t smem = bytes(tc);
    if (smem > 227 * 1024) SPY_FAIL("recurrence: a key size of %d does not fit a block's shared memory", A.dk);
    void (*kernel)(ScanArgs, int) = nullptr;
    const bool light = tc == 1 && nr <= 16;   // decoding: more blocks an SM, so that more of the state is on its way at a time
    switch (nr) {
        case 2: kernel = light ? scan_kernel<MODE, 2, true> : scan_kernel<MODE, 2, false>; break;
        case 4: kernel = light ? scan_kernel<MODE, 4, true> : scan_kernel<MODE, 4, false>; break;
        case 8: kernel = light ? scan_kernel<MODE, 8, true> : scan_kernel<MODE, 8, false>; break;
        case 16: kernel = light ? scan_kernel<MODE, 16, true> : scan_kernel<MODE, 16, false>; break;
        case 32: kernel = scan_kernel<MODE, 32, false>; break;
        default: kernel = scan_kernel<MODE, 64, false>; break;
    }
    if (smem > 48 * 1024) SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    spy_launch(kernel, dim3(num_seqs, A.H, tiles), dim3(THREADS), smem, stream, A, tc);
    SPY_CHECK_LAUNCH("recurrence scan");
    return 0;
}

static int launch_scan(int mode, ScanArgs& A, int num_seqs, int longest, cudaStream_t stream)
{
    if (num_seqs <= 0) return 0;
    if (A.H <= 0 || A.dk <= 0 || A.dv <= 0) SPY_FAIL("recurrence: heads %d, key size %d and value size %d must be positive", A.H, A.dk, A.dv);
    if (A.H > 65535) SPY_FAIL("recurrence: %d heads exceed the grid limit", A.H);
    if ((A.dv + CT - 1) / CT > 65535) SPY_FAIL("recurrence: a value size of %d exceeds the grid limit", A.dv);
    return mode == 0 ? launch_scan_mode<0>(A, num_seqs, longest, stream) : launch_scan_mode<1>(A, num_seqs, longest, stream);
}

// State record of one head, in floats.
extern "C" long long spy_mlstm_record(int dk, int dv) { return ((long long)dk * dv + (long long)((dv + CT - 1) / CT) * (dk + 1) + 3) / 4 * 4; }

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

// ---- what follows a recurrence: unit root mean square per head, a weight, a sigmoid gate -------------
template <typename TO>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ proj, long long ld, int off_g, const float* __restrict__ weight,
                                       TO* __restrict__ out, int H, int dv, float eps)
{
    __shared__ float scratch[33];
    pdl_enter();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) ss += src[c] * src[c];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const float* g = proj + (size_t)t * ld + off_g + h * dv;
    for (int c = threadIdx.x; c < dv; c += blockDim.x)
        out[((size_t)t * H + h) * dv + c] = from_f32<TO>(((src[c] * inv) * weight[h * dv + c]) * sigmoidf_(g[c]));
}

extern "C" int spy_gated_head_norm(const float* o, const float* proj, long long ld, int off_g, const float* weight, void* out, int out_dtype, int tokens,
                                   int H, int dv, float eps, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (H <= 0 || dv <= 0 || H > 65535) SPY_FAIL("gated_head_norm: %d heads of %d", H, dv);
    int threads = (dv + 31) / 32 * 32;
    threads = threads > 256 ? 256 : (threads < 32 ? 32 : threads);
    SPY_DISPATCH_DTYPE(out_dtype, TO, {
        spy_launch(gated_head_norm_kernel<TO>, dim3(tokens, H), dim3(threads), 0, stream, o, proj, ld, off_g, weight, (TO*)out, H, dv, eps);
    })
    SPY_CHECK_LAUNCH("gated_head_norm");
    return 0;
}

// out[t, j] = tanh(proj[t, off + j]) for j < n: the inner activation of a two-step (low-rank) projection.
template <typename TO>
__global__ void tanh_cols_kernel(const float* __restrict__ proj, long long ld, int off, int n, TO* __restrict__ out, long long total)
{
    pdl_enter();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const long long t = i / n;
        out[i] = from_f32<TO>(tanhf(proj[t * ld + off + (i - t * n)]));
    }
}

extern "C" int spy_tanh_cols(const float* proj, long long ld, int off, int n, void* out, int out_dtype, int tokens, cudaStream_t stream)
{
    if (tokens <= 0 || n <= 0) return 0;
    const long long total = (long long)tokens * n;
    long long blocks = (total + 255) / 256;
    const long long most = (long long)spy_sm_count() * 32;
    if (blocks > most) blocks = most;
    SPY_DISPATCH_DTYPE(out_dtype, TO, {
        spy_launch(tanh_cols_kernel<TO>, dim3((int)blocks), dim3(256), 0, stream, proj, ld, off, n, (TO*)out, total);
    })
    SPY_CHECK_LAUNCH("tanh_cols");
    return 0;
}
