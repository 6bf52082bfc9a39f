// Attention through a shared latent (keys and values of all heads are projections of one small vector per token, which is
// all the cache keeps, beside one rotated key part that the heads share).  Written in the absorbed form: with the per-head
// key projection U_k and value projection U_v of the latent c,
//     score = q_n . (U_k c) + q_r . k_r = (U_k^T q_n) . c + q_r . k_r,        o = U_v (sum_j p_j c_j),
// so the attention itself runs over ONE key/value head whose key is the cache row [c | k_r] and whose value is c, with the
// query [U_k^T q_n | rot(q_r)] per head, by the engine's ordinary attention kernels on a cache of one plane.  Here are the
// three steps around it:
//   latent_prep     RMS norms (32-bit statistics, plain weights) of the query latent and of the key/value latent, rotation
//                   of the shared key part, and the store of [c | k_r] into the token's cache row;
//   head_product    out[t, h, :N] = W_h^T in[t, h, :K] per head (32-bit sums), W given as [H][K][N]; used for the query's
//                   absorption (W = U_k as stored, plus the rotation of the `tail` that follows each head's K inputs) and
//                   for the value expansion (W = U_v transposed per head, plus an optional sigmoid gate on the result).
// Rotation: angle j of the (cos, sin) table turns the pair (j, j + r) ("half") or (2j, 2j + 1) ("interleaved") of the
// rotated part's first 2r elements; what lies beyond passes unchanged.
#include "common.cuh"

SPY_MODULE(spy_latent)

constexpr int PREP_THREADS = 128;
constexpr int TOK = 8;          // tokens a block of head_product takes (16 for prompts); a weight element is loaded once for all of them

// element j of the rotated vector x[0 .. n) at a position whose table row is cs (cos, sin pairs)
__device__ __forceinline__ float rotated(const float* x, int j, int rot_half, int interleaved, const float* cs)
{
    if (j >= 2 * rot_half) return x[j];
    int a, first;
    float u, v;
    if (interleaved) { a = j >> 1; first = (j & 1) == 0; u = x[2 * a]; v = x[2 * a + 1]; }
    else { a = j < rot_half ? j : j - rot_half; first = j < rot_half; u = x[a]; v = x[a + rot_half]; }
    const float c = cs[2 * a], s = cs[2 * a + 1];
    return first ? u * c - v * s : v * c + u * s;
}

template <typename TO, typename TC>
__global__ void __launch_bounds__(PREP_THREADS)
latent_prep_kernel(const float* __restrict__ fused, long long ld, int off_q, int q_rank, const float* __restrict__ wq, TO* __restrict__ cq_out,
                   int off_c, int kv_rank, const float* __restrict__ wc, int rot_dim, const float* __restrict__ rope, int rot_half, int table_rows,
                   int interleaved, const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                   int table_width, TC* __restrict__ pages, int page_size, int num_pages, int planes, float eps, int* status)
{
    extern __shared__ float sm[];           // rot_dim floats, then 33 of scratch
    pdl_enter();
    float* rot_s = sm;
    float* scratch = sm + rot_dim;
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* row = fused + (size_t)t * ld;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int i = tid; i < q_rank; i += PREP_THREADS) ss = fmaf(row[off_q + i], row[off_q + i], ss);
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = tid; i < q_rank; i += PREP_THREADS) cq_out[(size_t)t * q_rank + i] = from_f32<TO>((row[off_q + i] * inv) * wq[i]);
    }
    if (off_c < 0) return;
    const int pos = positions[t], seq = seq_of_token[t];
    const int lp = pos / page_size;
    const int page = (pos >= 0 && lp < table_width) ? block_table[(size_t)seq * table_width + lp] : -1;
    const bool page_ok = page >= 0 && page < num_pages;
    const bool pos_ok = rot_half == 0 || (pos >= 0 && pos < table_rows);
    if (!page_ok || !pos_ok) {
        if (tid == 0) report_status(status, page_ok ? SPY_STATUS_BAD_POSITION : SPY_STATUS_BAD_PAGE, t);
        return;
    }
    const int width = kv_rank + rot_dim;
    TC* dst = pages + (((size_t)page * planes) * page_size + pos % page_size) * width;     // plane 0 of the page's one key/value head
    float ss = 0.f;
    for (int i = tid; i < kv_rank; i += PREP_THREADS) ss = fmaf(row[off_c + i], row[off_c + i], ss);
    for (int j = tid; j < rot_dim; j += PREP_THREADS) rot_s[j] = row[off_c + kv_rank + j];
    ss = block_sum(ss, scratch);            // its barriers also publish rot_s
    const float inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    for (int i = tid; i < kv_rank; i += PREP_THREADS) dst[i] = from_f32<TC>((row[off_c + i] * inv) * wc[i]);
    const float* cs = rope + (size_t)(rot_half ? pos : 0) * rot_half * 2;
    for (int j = tid; j < rot_dim; j += PREP_THREADS) dst[kv_rank + j] = from_f32<TC>(rotated(rot_s, j, rot_half, interleaved, cs));
}

// fused [T, ld] float32: the query latent before its norm at off_q (q_rank columns; 0: none), the key/value latent and the
// shared key part at off_c (kv_rank + rot_dim columns; off_c < 0: this layer stores nothing).  cq_out [T, q_rank].
// pages [num_pages][planes][1][page_size][kv_rank + rot_dim].  rope [table_rows][rot_half][2] or null with rot_half 0.
extern "C" int spy_latent_prep(const float* fused, long long ld, int off_q, int q_rank, const float* wq, void* cq_out, int out_dtype, int off_c,
                               int kv_rank, const float* wc, int rot_dim, const float* rope, int rot_half, int table_rows, int interleaved,
                               const int* positions, const int* seq_of_token, const int* block_table, int table_width, void* pages, int cache_dtype,
                               int page_size, int num_pages, int planes, float eps, int tokens, int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (q_rank < 0 || (q_rank > 0 && (wq == nullptr || cq_out == nullptr))) SPY_FAIL("latent_prep: the query latent needs its norm weight and a place to go");
    if (off_c >= 0) {
        if (kv_rank <= 0 || rot_dim < 0 || wc == nullptr || pages == nullptr || block_table == nullptr) SPY_FAIL("latent_prep: storing needs the latent's size, its norm weight, pages and a block table");
        if (2 * rot_half > rot_dim || (rot_half > 0 && rope == nullptr)) SPY_FAIL("latent_prep: %d rotated pairs do not fit a rotated part of %d", rot_half, rot_dim);
        if (page_size <= 0 || num_pages <= 0 || table_width <= 0 || (planes != 1 && planes != 2)) SPY_FAIL("latent_prep: page_size, num_pages, table_width must be positive and planes 1 or 2");
    }
    const size_t smem = (size_t)((rot_dim > 0 ? rot_dim : 0) + 33) * sizeof(float);
    SPY_DISPATCH_DTYPE(out_dtype, TO, {
        SPY_DISPATCH_DTYPE(cache_dtype, TC, {
            spy_launch(latent_prep_kernel<TO, TC>, dim3(tokens), dim3(PREP_THREADS), smem, stream, fused, ld, off_q, q_rank, wq, (TO*)cq_out, off_c, kv_rank, wc,
                       rot_dim, rope, rot_half, table_rows, interleaved, positions, seq_of_token, block_table, table_width, (TC*)pages, page_size, num_pages,
                       planes, eps, status);
        })
    })
    SPY_CHECK_LAUNCH("latent_prep");
    return 0;
}

struct HeadProductArgs {
    const void* in;  long long in_ld;  int in_head_stride;  int K;
    const void* W;   int N;
    void* out;       long long out_ld; int out_head_stride;
    int tail;                 // elements after each head's K inputs that go, rotated, to the columns after its N outputs
    const float* rope; int rot_half, table_rows, interleaved; const int* positions;
    const float* gate; long long gate_ld; int gate_off;      // null, or out *= sigmoid(gate[t, gate_off + h * N + n])
    int T;
    int* status;
};

constexpr int KC = 32;          // weight rows staged at a time
constexpr int NC = 128;         // output columns a pass of a block takes: one a thread

// A block takes NT tokens of one head: their inputs wait in shared memory as [input element][token], so that a thread
// reads four tokens' values at a time, and a weight element is loaded once for all NT tokens.  The weights come through
// shared memory too, KC rows of the block's 128 columns at a time, every thread's loads of a chunk under way together
// (a thread that fetched its column's weights one after the other from L2 spent its time waiting for them).  A token's
// sum runs over the inputs in their order whatever NT is.
template <typename TA, typename TW, int NT>
__global__ void __launch_bounds__(128) head_product_kernel(HeadProductArgs A)
{
    extern __shared__ __align__(16) float in_s[];        // [K + tail][NT + 4] (the pad spreads a column's stores over the banks), then the weights' chunk [KC][NC]
    constexpr int LD = NT + 4;
    pdl_enter();
    const int t0 = blockIdx.x * NT, h = blockIdx.y, tid = threadIdx.x;
    const int n_tok = min(NT, A.T - t0), KT = A.K + A.tail;
    float* w_s = in_s + (size_t)KT * LD;
    const TA* in = (const TA*)A.in;
    TA* out = (TA*)A.out;
    for (int first = tid; first < NT * KT; first += 8 * 128) {        // eight loads a thread under way at a time
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int idx = first + j * 128, u = idx / KT, k = idx - u * KT;
            v[j] = (idx < NT * KT && u < n_tok) ? to_f32(in[(size_t)(t0 + u) * A.in_ld + (size_t)h * A.in_head_stride + k]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int idx = first + j * 128, u = idx / KT, k = idx - u * KT;
            if (idx < NT * KT) in_s[k * LD + u] = v[j];
        }
    }
    const TW* W = (const TW*)A.W + (size_t)h * A.K * A.N;
    for (int n0 = 0; n0 < A.N; n0 += NC) {
        const int n = n0 + tid, cols = min(NC, A.N - n0);
        float acc[NT];
#pragma unroll
        for (int u = 0; u < NT; ++u) acc[u] = 0.f;
        for (int k0 = 0; k0 < A.K; k0 += KC) {
            const int kc = min(KC, A.K - k0);
            __syncthreads();                             // the chunk before has been used (and, the first time, in_s is written)
            if (tid < cols) {
#pragma unroll 8
                for (int r = 0; r < kc; ++r) w_s[r * NC + tid] = to_f32(W[(size_t)(k0 + r) * A.N + n]);
            }
            __syncthreads();
            if (tid < cols) {
                for (int r = 0; r < kc; ++r) {
                    const float w = w_s[r * NC + tid];
#pragma unroll
                    for (int u = 0; u < NT; u += 4) {
                        const float4 x = *reinterpret_cast<const float4*>(in_s + (k0 + r) * LD + u);
                        acc[u] = fmaf(w, x.x, acc[u]);
                        acc[u + 1] = fmaf(w, x.y, acc[u + 1]);
                        acc[u + 2] = fmaf(w, x.z, acc[u + 2]);
                        acc[u + 3] = fmaf(w, x.w, acc[u + 3]);
                    }
                }
            }
        }
        if (tid >= cols) continue;
#pragma unroll
        for (int u = 0; u < NT; ++u) {
            if (u < n_tok) {
                float r = acc[u];
                if (A.gate != nullptr) {
                    const float g = A.gate[(size_t)(t0 + u) * A.gate_ld + A.gate_off + (size_t)h * A.N + n];
                    r *= 1.0f / (1.0f + expf(-g));
                }
                out[(size_t)(t0 + u) * A.out_ld + (size_t)h * A.out_head_stride + n] = from_f32<TA>(r);
            }
        }
    }
    if (A.tail > 0) {
        for (int idx = tid; idx < n_tok * A.tail; idx += 128) {
            const int u = idx / A.tail, j = idx - u * A.tail;
            const int pos = A.positions[t0 + u];
            if (A.rot_half > 0 && (pos < 0 || pos >= A.table_rows)) {
                report_status(A.status, SPY_STATUS_BAD_POSITION, t0 + u);
                continue;
            }
            const float* cs = A.rope + (size_t)(A.rot_half ? pos : 0) * A.rot_half * 2;
            // element j of the rotated tail, read from the [element][token] layout
            float r;
            if (j >= 2 * A.rot_half) {
                r = in_s[(A.K + j) * LD + u];
            } else {
                int a, first;
                float x, y;
                if (A.interleaved) { a = j >> 1; first = (j & 1) == 0; x = in_s[(A.K + 2 * a) * LD + u]; y = in_s[(A.K + 2 * a + 1) * LD + u]; }
                else { a = j < A.rot_half ? j : j - A.rot_half; first = j < A.rot_half; x = in_s[(A.K + a) * LD + u]; y = in_s[(A.K + a + A.rot_half) * LD + u]; }
                const float c = cs[2 * a], sn = cs[2 * a + 1];
                r = first ? x * c - y * sn : y * c + x * sn;
            }
            out[(size_t)(t0 + u) * A.out_ld + (size_t)h * A.out_head_stride + A.N + j] = from_f32<TA>(r);
        }
    }
}

// in [T, in_ld]: head h's K inputs (and `tail` more) start at column h * in_head_stride.  W [H][K][N] (w_dtype).
// out [T, out_ld]: head h's N results (and the rotated tail) start at column h * out_head_stride.  in and out have act_dtype.
extern "C" int spy_head_product(const void* in, long long in_ld, int in_head_stride, int K, const void* W, int w_dtype, int N, void* out, long long out_ld,
                                int out_head_stride, int act_dtype, int tail, const float* rope, int rot_half, int table_rows, int interleaved,
                                const int* positions, const float* gate, long long gate_ld, int gate_off, int tokens, int heads, int* status,
                                cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || K <= 0 || N <= 0 || tail < 0) SPY_FAIL("head_product: %d heads, K %d, N %d, tail %d", heads, K, N, tail);
    if (tail > 0 && (positions == nullptr || 2 * rot_half > tail || (rot_half > 0 && rope == nullptr))) SPY_FAIL("head_product: the rotated tail needs positions and a table that fits it");
    if (in_head_stride < K + tail || out_head_stride < N + tail) SPY_FAIL("head_product: a head's columns overlap the next head's");
    const int nt = tokens >= 256 ? 16 : TOK;      // prompts: more tokens share a weight element (32 of them cost registers, hence resident blocks, and were slower)
    const size_t smem = ((size_t)(nt + 4) * (K + tail) + (size_t)KC * NC) * sizeof(float);
    if (smem > 160 * 1024) SPY_FAIL("head_product: %d inputs a head do not fit a block's shared memory", K + tail);
    HeadProductArgs A = {in, in_ld, in_head_stride, K, W, N, out, out_ld, out_head_stride, tail, rope, rot_half, table_rows, interleaved, positions,
                         gate, gate_ld, gate_off, tokens, status};
    SPY_DISPATCH_DTYPE(act_dtype, TA, {
        SPY_DISPATCH_DTYPE(w_dtype, TW, {
            auto kernel = nt == 16 ? head_product_kernel<TA, TW, 16> : head_product_kernel<TA, TW, TOK>;
            if (smem > 48 * 1024) SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            spy_launch(kernel, dim3((tokens + nt - 1) / nt, heads), dim3(128), smem, stream, A);
        })
    })
    SPY_CHECK_LAUNCH("head_product");
    return 0;
}
