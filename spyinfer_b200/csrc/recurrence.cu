// Linear recurrences over a matrix state per (request, head), carried from token to token in 32-bit:
//   * the gated matrix memory (mLSTM):       S = a S + b k v^T,  n = a n + b k,  o = S^T q / (max(|n . q|, exp(-m)) + 1e-6)
//                                            with log gates i, f, the running maximum m' = max(f + m, i) (m starts at 0),
//                                            a = exp(f + m - m'), b = exp(i - m');
//   * the generalised delta rule:            S = diag(w) S - (r u)(u^T S) + k v^T,  o = S^T q,  u = k / sqrt(sum k^2 + 1e-6),
//                                            both terms reading the old S, w a decay and r a removal rate per key channel;
// and what follows both: each head's output divided by its root mean square, times a weight, times a sigmoid gate.
//
// One kernel serves prompt portions and decoding: a block owns CT = 32 value columns of one (request, head), holds its
// [dk x 32] tile of S in shared memory and walks the request's tokens of this step in order.  The columns of S do not
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

// Sum over the block of one value per thread, through `part` (one float a warp); every thread gets the result.
// Must be followed by a barrier before `part` is written again.
__device__ __forceinline__ float block_total(float v, float* part)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_sum(v);
    if (lane == 0) part[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nwarps; ++w) t += part[w];
    return t;
}

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

template <int MODE>   // 0: gated matrix memory, 1: delta rule
__global__ void __launch_bounds__(256) scan_kernel(ScanArgs A)
{
    extern __shared__ float sm[];
    pdl_enter();
    const int dk = A.dk, dv = A.dv, H = A.H;
    const int R = blockDim.x / CT;                 // row groups
    float* S = sm;                                 // [dk][CT]
    float* k_s = S + (size_t)dk * CT;              // dk
    float* q_s = k_s + dk;                         // dk
    float* x1_s = q_s + dk;                        // dk: mLSTM n; delta removal rate
    float* x2_s = x1_s + dk;                       // dk: delta decay
    float* red = x2_s + dk;                        // [R][CT]
    float* red2 = red + R * CT;                    // [R][CT]
    float* part = red2 + R * CT;                   // 32

    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CT;
    const int tid = threadIdx.x, c = tid % CT, rg = tid / CT;
    const bool col_ok = c0 + c < dv;
    const int t0 = A.q_start[seq], t1 = A.q_start[seq + 1];
    if (t0 >= t1) return;
    const int slot = A.state_slot[seq];
    if (slot < 0 || slot >= A.num_slots) {
        if (tid == 0) report_status(A.status, SPY_STATUS_BAD_PAGE, t0);
        return;
    }
    float* st = A.state + ((size_t)slot * H + h) * A.record;
    for (int r = rg; r < dk; r += R) S[r * CT + c] = col_ok ? st[(size_t)r * dv + c0 + c] : 0.f;
    float m = 0.f;
    float* st_nm = st + (size_t)dk * dv + (size_t)blockIdx.z * (dk + 1);      // this tile's own copy of n and m
    if (MODE == 0) {
        for (int r = tid; r < dk; r += blockDim.x) x1_s[r] = st_nm[r];
        m = st_nm[dk];
    }
    __syncthreads();

    for (int t = t0; t < t1; ++t) {
        const float* row = A.proj + (size_t)t * A.ld;
        const float v_c = col_ok ? row[A.off_v + h * dv + c0 + c] : 0.f;
        if (MODE == 0) {
            // gates, by every thread alike (two numbers a head)
            const float ig = A.cap * tanhf((row[A.off_x1 + h] + A.bias1[h]) / A.cap);
            const float fg = log_sigmoidf_(A.cap * tanhf((row[A.off_x2 + h] + A.bias2[h]) / A.cap));
            const float m_new = fmaxf(fg + m, ig);
            const float a = expf(fg + m - m_new), b = expf(ig - m_new);
            m = m_new;
            float nq = 0.f;
            for (int r = tid; r < dk; r += blockDim.x) {
                const float kr = row[A.off_k + h * dk + r], qr = row[A.off_q + h * dk + r] * A.q_scale;
                const float n = a * x1_s[r] + b * kr;
                k_s[r] = kr;
                q_s[r] = qr;
                x1_s[r] = n;
                nq += n * qr;
            }
            nq = block_total(nq, part);            // its barrier also publishes k_s and q_s
            float acc = 0.f;
            for (int r = rg; r < dk; r += R) {
                const float s = a * S[r * CT + c] + (b * k_s[r]) * v_c;
                S[r * CT + c] = s;
                acc = fmaf(s, q_s[r], acc);
            }
            red[rg * CT + c] = acc;
            __syncthreads();
            if (rg == 0 && col_ok) {
                float o = 0.f;
                for (int g = 0; g < R; ++g) o += red[g * CT + c];
                A.out[(size_t)t * H * dv + h * dv + c0 + c] = o / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
            }
            __syncthreads();                       // k_s, q_s, red and part are rewritten by the next token
        } else {
            float ksq = 0.f;
            for (int r = tid; r < dk; r += blockDim.x) {
                const int col = h * dk + r;
                const float kr = row[A.off_k + col];
                k_s[r] = kr;
                q_s[r] = row[A.off_q + col];
                x1_s[r] = sigmoidf_(row[A.off_x1 + col] + A.bias1[col]);
                x2_s[r] = expf(-0.60653065971263342f * sigmoidf_(A.extra[(size_t)t * H * dk + col] + A.bias2[col]));   // exp(-1/2) = 0.6065...
                ksq += kr * kr;
            }
            ksq = block_total(ksq, part);          // its barrier also publishes the vectors
            const float inv = 1.0f / sqrtf(ksq + 1e-6f);
            float us = 0.f;
            for (int r = rg; r < dk; r += R) us = fmaf(k_s[r] * inv, S[r * CT + c], us);
            red[rg * CT + c] = us;
            __syncthreads();
            us = 0.f;
            for (int g = 0; g < R; ++g) us += red[g * CT + c];
            float acc = 0.f;
            for (int r = rg; r < dk; r += R) {
                const float u = k_s[r] * inv;
                const float s = x2_s[r] * S[r * CT + c] - (x1_s[r] * u) * us + k_s[r] * v_c;
                S[r * CT + c] = s;
                acc = fmaf(s, q_s[r], acc);
            }
            red2[rg * CT + c] = acc;
            __syncthreads();
            if (rg == 0 && col_ok) {
                float o = 0.f;
                for (int g = 0; g < R; ++g) o += red2[g * CT + c];
                A.out[(size_t)t * H * dv + h * dv + c0 + c] = o;
            }
            __syncthreads();
        }
    }
    if (col_ok)
        for (int r = rg; r < dk; r += R) st[(size_t)r * dv + c0 + c] = S[r * CT + c];
    if (MODE == 0) {
        for (int r = tid; r < dk; r += blockDim.x) st_nm[r] = x1_s[r];
        if (tid == 0) st_nm[dk] = m;
    }
}

static int launch_scan(int mode, ScanArgs& A, int num_seqs, cudaStream_t stream)
{
    if (num_seqs <= 0) return 0;
    if (A.H <= 0 || A.dk <= 0 || A.dv <= 0) SPY_FAIL("recurrence: heads %d, key size %d and value size %d must be positive", A.H, A.dk, A.dv);
    if (A.H > 65535) SPY_FAIL("recurrence: %d heads exceed the grid limit", A.H);
    const int tiles = (A.dv + CT - 1) / CT;
    if (tiles > 65535) SPY_FAIL("recurrence: a value size of %d exceeds the grid limit", A.dv);
    const int threads = A.dk >= 64 ? 256 : 128;
    const int R = threads / CT;
    const size_t smem = ((size_t)A.dk * CT + 4 * (size_t)A.dk + 2 * (size_t)R * CT + 64) * sizeof(float);
    if (smem > 227 * 1024) SPY_FAIL("recurrence: a key size of %d does not fit a block's shared memory", A.dk);
    auto kernel = mode == 0 ? scan_kernel<0> : scan_kernel<1>;
    if (smem > 48 * 1024) SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    spy_launch(kernel, dim3(num_seqs, A.H, tiles), dim3(threads), smem, stream, A);
    SPY_CHECK_LAUNCH("recurrence scan");
    return 0;
}

// State record of one head, in floats.
extern "C" long long spy_mlstm_record(int dk, int dv) { return ((long long)dk * dv + (long long)((dv + CT - 1) / CT) * (dk + 1) + 3) / 4 * 4; }

extern "C" int spy_mlstm_scan(const float* proj, long long ld, int off_q, int off_k, int off_v, int off_i, int off_f, const float* bias_i, const float* bias_f,
                              float* state, int num_slots, const int* q_start, const int* state_slot, int num_seqs, float* out, int H, int dk, int dv,
                              float q_scale, float cap, int* status, cudaStream_t stream)
{
    if (!(cap > 0.f)) SPY_FAIL("mlstm: the gates' cap must be positive");
    ScanArgs A = {proj, ld, off_q, off_k, off_v, off_i, off_f, nullptr, bias_i, bias_f, state, spy_mlstm_record(dk, dv), num_slots, q_start, state_slot, out,
                  H, dk, dv, q_scale, cap, status};
    return launch_scan(0, A, num_seqs, stream);
}

extern "C" int spy_delta_scan(const float* proj, long long ld, int off_r, int off_k, int off_v, int off_a, const float* decay_pre, const float* bias_a,
                              const float* decay_offset, float* state, int num_slots, const int* q_start, const int* state_slot, int num_seqs, float* out,
                              int H, int dk, int* status, cudaStream_t stream)
{
    ScanArgs A = {proj, ld, off_r, off_k, off_v, off_a, 0, decay_pre, bias_a, decay_offset, state, (long long)dk * dk, num_slots, q_start, state_slot, out,
                  H, dk, dk, 1.0f, 1.0f, status};
    return launch_scan(1, A, num_seqs, stream);
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
