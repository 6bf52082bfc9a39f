// Attention over a window of recent keys plus one pooled key and value for every block of tokens that
// lies wholly before the window, all under one softmax; and the kernel that makes the pooled entries.
//
// A query at position p of sequence s sees
//   * the keys j with p - window < j <= p, from the token cache (page block_table[s, j / page_size], slot j % page_size);
//   * the pooled entries b with b * pool + pool - 1 <= p - window, from the pooled cache (one entry for every `pool`
//     tokens: page pool_table[s, b / page_size], slot b % page_size), entry b being the mean of the keys (values) of the
//     positions b * pool .. b * pool + pool - 1 as the token cache holds them.
// A token that has left the window while its block is not yet complete enough to be seen is seen by nobody.
// kv head = head / (nh / nkv); score = (q . k) * scale; p = exp(score - max) / sum; o = sum p v.
//
// This is the plain kernel (one block per (query token, head), everything in 32-bit, any head size that is a multiple
// of 4, any page size, 32-bit or bfloat16 storage); it serves prompt portions and decoding alike.  The keys of a query
// form one list, pooled entries first, and are processed in chunks of 128 of that list, so a query's result does not
// depend on how the batch was cut.
#include "common.cuh"

SPY_MODULE(spy_attention_pool)

constexpr int CHUNK = 128;

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4])
    {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
};

// ---- pooled entries ------------------------------------------------------------------------------
// One block per (16 tokens of the batch, K or V, kv head): it looks through its tokens, and for each whose position ends a
// block of `pool` tokens it writes that block's entry.  The block's threads form row groups: group y adds the rows y,
// y + groups, ... of the pooled block (so that their loads are in flight together), and the groups' sums are added in the
// order of the groups.
constexpr int POOL_TOKENS = 16;

template <typename TC>
__global__ void pool_store_kernel(const TC* __restrict__ pages, int num_pages, const int* __restrict__ block_table, TC* __restrict__ pooled,
                                  int num_pooled_pages, const int* __restrict__ pool_table, int table_width, int page_size, int nkv, int hd, int pool,
                                  const int* __restrict__ positions, const int* __restrict__ seq_of_token, int tokens, int* status)
{
    extern __shared__ float part[];   // [groups][hd]
    __shared__ int pos_s[POOL_TOKENS];
    pdl_enter();
    const int which = blockIdx.y / nkv, kvh = blockIdx.y % nkv;
    const int groups = blockDim.y, y = threadIdx.y;
    const int first = blockIdx.x * POOL_TOKENS, flat = threadIdx.y * blockDim.x + threadIdx.x;
    if (flat < POOL_TOKENS) pos_s[flat] = first + flat < tokens ? positions[first + flat] : -2;     // all at once, not one round trip a token
    __syncthreads();
    for (int t = first; t < min(tokens, first + POOL_TOKENS); ++t) {
        const int pos = pos_s[t - first];
        if ((pos + 1) % pool != 0) continue;          // the same for every thread
        const int b = (pos + 1) / pool - 1, seq = seq_of_token[t];
        const int* bt = block_table + (size_t)seq * table_width;
        const int lp_out = b / page_size;
        const int out_page = lp_out < table_width ? pool_table[(size_t)seq * table_width + lp_out] : -1;
        if (out_page < 0 || out_page >= num_pooled_pages) {
            if (threadIdx.x == 0 && threadIdx.y == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
            continue;
        }
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {
            float sum = 0.f;
            for (int j0 = b * pool + y; j0 <= pos; j0 += 4 * groups) {      // four rows' pages are looked up, then their loads are under way together
                const TC* src[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j0 + e * groups;
                    src[e] = nullptr;
                    if (j > pos) continue;
                    const int lp = j / page_size;
                    const int page = lp < table_width ? bt[lp] : -1;
                    if (page < 0 || page >= num_pages) report_status(status, SPY_STATUS_BAD_PAGE, t);
                    else src[e] = pages + ((((size_t)page * 2 + which) * nkv + kvh) * page_size + j % page_size) * hd + d;
                }
                float x[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) x[e] = src[e] != nullptr ? to_f32(*src[e]) : 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) sum += x[e];
            }
            part[y * hd + d] = sum;
        }
        __syncthreads();
        if (y == 0) {
            TC* dst = pooled + ((((size_t)out_page * 2 + which) * nkv + kvh) * page_size + b % page_size) * hd;
            const float inv = 1.0f / (float)pool;
            for (int d = threadIdx.x; d < hd; d += blockDim.x) {
                float sum = 0.f;
                for (int g = 0; g < groups; ++g) sum += part[g * hd + d];
                dst[d] = from_f32<TC>(sum * inv);
            }
        }
        __syncthreads();                              // part is rewritten for the block's next token
    }
}

extern "C" int spy_pool_store(const void* pages, int num_pages, const int* block_table, void* pooled, int num_pooled_pages, const int* pool_table,
                              int table_width, int page_size, int nkv, int hd, int cache_dtype, int pool, const int* positions, const int* seq_of_token,
                              int tokens, int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (pool <= 0 || page_size <= 0 || nkv <= 0 || hd <= 0 || table_width <= 0) SPY_FAIL("pool_store: pool, page_size, heads, head size and table width must be positive");
    if (2 * nkv > 65535) SPY_FAIL("pool_store: %d key/value heads exceed the grid limit", nkv);
    int tx = hd <= 32 ? 32 : 64;       // few threads along the head, many row groups: the rows' loads are what takes the time
    int ty = 256 / tx;
    while (ty > 1 && ty > pool) ty /= 2;
    const size_t smem = (size_t)ty * hd * sizeof(float);
    if (smem > 48 * 1024) SPY_FAIL("pool_store: a head size of %d does not fit", hd);
    SPY_DISPATCH_DTYPE(cache_dtype, TC, {
        spy_launch(pool_store_kernel<TC>, dim3((tokens + POOL_TOKENS - 1) / POOL_TOKENS, 2 * nkv), dim3(tx, ty), smem, stream, (const TC*)pages, num_pages,
                   block_table, (TC*)pooled, num_pooled_pages, pool_table, table_width, page_size, nkv, hd, pool, positions, seq_of_token, tokens, status);
    })
    SPY_CHECK_LAUNCH("pool_store");
    return 0;
}

// ---- attention -------------------------------------------------------------------------------------
template <typename TA, typename TC>
__global__ void __launch_bounds__(CHUNK)
attention_pool_kernel(const TA* __restrict__ q, long long q_row_stride, TA* __restrict__ out, const TC* __restrict__ pages, int num_pages,
                      const int* __restrict__ block_table, const TC* __restrict__ pooled, int num_pooled_pages, const int* __restrict__ pool_table,
                      int table_width, int page_size, int nh, int nkv, int hd, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      int window, int pool, float scale, const float* __restrict__ lse, int* status)
{
    extern __shared__ float smem[];
    pdl_enter();
    float* q_s = smem;                                   // hd
    float* p_s = q_s + hd;                               // CHUNK
    const TC** row_s = (const TC**)(p_s + CHUNK);        // CHUNK pointers to K rows; 8-byte aligned: hd % 4 == 0, CHUNK even
    float* scratch = (float*)(row_s + CHUNK);            // 33

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int kvh = h / (nh / nkv);
    const int* bt = block_table + (size_t)seq * table_width;
    const int* pt = pool_table ? pool_table + (size_t)seq * table_width : nullptr;
    const long long v_offset = (long long)nkv * page_size * hd;  // from a K row to its V row, in both caches

    const int lo = max(0, pos - window + 1);
    const int nb = (pool > 0 && pos - window + 1 >= pool) ? (pos - window + 1) / pool : 0;   // blocks that end at or before pos - window
    // lse given: another kernel has done the window's keys (its normalised result is in `out`, the logarithm of its sum of
    // exponentials in lse); only the pooled entries are walked here and merged with that result at the end
    const int total = lse != nullptr ? nb : nb + (pos - lo + 1);
    if (total == 0) return;

    const TA* q_row = q + (size_t)t * q_row_stride + (size_t)h * hd;
    for (int d = tid; d < hd; d += CHUNK) q_s[d] = to_f32(q_row[d]);

    float m = -INFINITY, l = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};  // dims tid, tid+128, tid+256, tid+384
    __syncthreads();

    for (int c0 = 0; c0 < total; c0 += CHUNK) {
        const int idx = c0 + tid;
        bool valid = idx < total;
        const TC* row = nullptr;
        if (valid) {
            const bool is_pooled = idx < nb;
            const int e = is_pooled ? idx : lo + (idx - nb);     // entry of the pooled cache, or position in the token cache
            const int lp = e / page_size;
            const int page = lp < table_width ? (is_pooled ? pt[lp] : bt[lp]) : -1;
            if (page < 0 || page >= (is_pooled ? num_pooled_pages : num_pages)) {
                report_status(status, SPY_STATUS_BAD_PAGE, t);
                valid = false;
            } else {
                row = (is_pooled ? pooled : pages) + ((((long long)page * 2) * nkv + kvh) * page_size + e % page_size) * hd;
            }
        }
        float s = -INFINITY;
        if (valid) {
            float dot = 0.f;
            for (int d = 0; d < hd; d += 4) {
                float kv[4];
                Vec4<TC>::load(row + d, kv);
                dot = fmaf(q_s[d], kv[0], dot);
                dot = fmaf(q_s[d + 1], kv[1], dot);
                dot = fmaf(q_s[d + 2], kv[2], dot);
                dot = fmaf(q_s[d + 3], kv[3], dot);
            }
            s = dot * scale;
        }
        const float chunk_max = block_max(s, scratch);
        const float m_new = fmaxf(m, chunk_max);
        if (m_new == -INFINITY) continue;  // every key of the chunk was refused: nothing to add (uniform over the block)
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
        p_s[tid] = p;
        row_s[tid] = row;
        const float chunk_sum = block_sum(p, scratch);  // its barriers also publish p_s and row_s
        l = l * alpha + chunk_sum;
        m = m_new;
        const int count = min(CHUNK, total - c0);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int d = tid + r * CHUNK;
            if (d < hd) {
                float a = acc[r] * alpha;
                for (int jj = 0; jj < count; ++jj)
                    if (row_s[jj] != nullptr) a = fmaf(p_s[jj], to_f32(row_s[jj][v_offset + d]), a);
                acc[r] = a;
            }
        }
        __syncthreads();  // p_s and row_s are rewritten by the next chunk
    }
    TA* o_row = out + ((size_t)t * nh + h) * hd;
    if (lse != nullptr) {
        const float lw = lse[(size_t)t * nh + h];
        const float top = fmaxf(lw, m);
        if (top == -INFINITY) return;
        const float fw = lw == -INFINITY ? 0.f : expf(lw - top), fp = m == -INFINITY ? 0.f : expf(m - top);
        const float inv = 1.0f / (fw + l * fp);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int d = tid + r * CHUNK;
            if (d < hd) o_row[d] = from_f32<TA>((to_f32(o_row[d]) * fw + acc[r] * fp) * inv);
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int d = tid + r * CHUNK;
        if (d < hd) o_row[d] = from_f32<TA>(l > 0.f ? acc[r] / l : 0.f);
    }
}

// q: [T, ...] rows of q_row_stride elements whose first nh*hd elements are the query heads; out: [T, nh*hd];
// pages / pooled: caches [pages][2][nkv][page_size][hd] of cache_dtype with a block table [S, table_width] each
// (pool == 0: no pooled entries, pooled and pool_table may be null).  lse (null, or [T, nh] float32): the window's keys
// have been done by another kernel, which left its normalised result in out and the natural logarithm of each row's sum of
// exponentials in lse; this call then adds the pooled entries to that softmax and rewrites out.
extern "C" int spy_attention_pool(const void* q, long long q_row_stride, void* out, int act_dtype, const void* pages, int num_pages,
                                  const int* block_table, const void* pooled, int num_pooled_pages, const int* pool_table, int cache_dtype,
                                  int table_width, int page_size, int nh, int nkv, int hd, const int* positions, const int* seq_of_token, int tokens,
                                  int window, int pool, float scale, const float* lse, int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (lse != nullptr && pool <= 0) return 0;   // nothing to merge
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) SPY_FAIL("attention: %d query heads do not group over %d key/value heads", nh, nkv);
    if (hd <= 0 || hd % 4 != 0 || hd > 4 * CHUNK) SPY_FAIL("attention: head_dim %d must be a multiple of 4, at most %d", hd, 4 * CHUNK);
    if (page_size <= 0 || num_pages <= 0 || table_width <= 0) SPY_FAIL("attention: page_size, num_pages and table_width must be positive");
    if (window <= 0) SPY_FAIL("attention: window %d must be positive", window);
    if (pool < 0 || (pool > 0 && (pooled == nullptr || pool_table == nullptr || num_pooled_pages <= 0))) SPY_FAIL("attention: pooled entries need their cache and block table");
    if (nh > 65535) SPY_FAIL("attention: %d heads exceed the grid limit", nh);
    const size_t smem = (size_t)(hd + CHUNK + 33) * sizeof(float) + (size_t)CHUNK * sizeof(void*);
    dim3 grid(tokens, nh);
    SPY_DISPATCH_DTYPE(act_dtype, TA, {
        SPY_DISPATCH_DTYPE(cache_dtype, TC, {
            spy_launch(attention_pool_kernel<TA, TC>, grid, dim3(CHUNK), smem, stream, (const TA*)q, q_row_stride, (TA*)out, (const TC*)pages, num_pages,
                       block_table, (const TC*)pooled, num_pooled_pages, pool_table, table_width, page_size, nh, nkv, hd, positions, seq_of_token, window,
                       pool, scale, lse, status);
        })
    })
    SPY_CHECK_LAUNCH("attention_pool");
    return 0;
}
