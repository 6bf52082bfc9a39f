// The residual sum of a block whose norm sits on the sublayer's OUTPUT:  h += rms_norm(y) * w,  h the 32-bit residual stream.
//   v   = y[row], itself possibly a sum of split-K partial products            32-bit sums
//   h[row] += v * (1 / sqrt(mean(v^2) + eps)) * w                              32-bit statistics; w as stored or as (offset + w)
//   copy[row] = h[row] in the activations' type                                what the next sublayer's products read (optional)
// With y absent the kernel only makes the copy (the embedding's rows for the first sublayer).
// One block a row.  Rows of up to 16 K elements (a multiple of 4) stay in registers; other rows wait in shared memory
// between the two passes.
#include "common.cuh"

SPY_MODULE(spy_residual_norm)

template <typename TY, typename TW, typename TC>
__global__ void __launch_bounds__(256) residual_norm_kernel(float* __restrict__ h, const TY* __restrict__ y, int splits, long long split_stride,
                                                            const TW* __restrict__ w, float w_offset, TC* __restrict__ copy, int len, float eps)
{
    extern __shared__ float row_buf[];   // len floats, then 33 of scratch
    pdl_enter();
    float* scratch = row_buf + len;
    const size_t base = (size_t)blockIdx.x * len;
    if (y != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < len; i += blockDim.x) {
            float v = 0.f;
            for (int s = 0; s < splits; ++s) v += to_f32(y[(size_t)s * split_stride + base + i]);   // the parts in their order
            row_buf[i] = v;
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)len + eps);
        for (int i = threadIdx.x; i < len; i += blockDim.x) {
            const float r = h[base + i] + (row_buf[i] * inv) * (w_offset + to_f32(w[i]));
            h[base + i] = r;
            if (copy != nullptr) copy[base + i] = from_f32<TC>(r);
        }
    } else if (copy != nullptr) {
        for (int i = threadIdx.x; i < len; i += blockDim.x) copy[base + i] = from_f32<TC>(h[base + i]);
    }
}

template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4])
    {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Quad<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4])
    {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4])
    {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<uint32_t*>(&a);
        x.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

// Rows whose length is a multiple of 4 and at most 16 K stay in registers: a thread owns NQ quads of the row (quad
// tid + j * blockDim.x), the weight's quads are loaded before the wait for the kernels ahead, the stream's and every
// part's loads are under way together, and the sums over the parts keep their order.
template <typename TY, typename TW, typename TC, int NQ, int MAXT>
__global__ void __launch_bounds__(MAXT) residual_norm_row_kernel(float* __restrict__ h, const TY* __restrict__ y, int splits, long long split_stride,
                                                                 const TW* __restrict__ w, float w_offset, TC* __restrict__ copy, int len, float eps)
{
    __shared__ float scratch[33];
    pdl_launch_dependents();
    float wv[NQ][4];
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int i = 4 * ((int)threadIdx.x + j * (int)blockDim.x);
        if (i < len) Quad<TW>::load(w + i, wv[j]);
    }
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * len;
    float hv[NQ][4], v[NQ][4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int i = 4 * ((int)threadIdx.x + j * (int)blockDim.x);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[j][e] = 0.f;
        if (i < len) {
            Quad<float>::load(h + base + i, hv[j]);
            for (int s0 = 0; s0 < splits; s0 += 4) {
                float d[4][4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (s0 + k < splits) Quad<TY>::load(y + (size_t)(s0 + k) * split_stride + base + i, d[k]);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (s0 + k < splits) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[j][e] += d[k][e];
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[j][e], v[j][e], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)len + eps);
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int i = 4 * ((int)threadIdx.x + j * (int)blockDim.x);
        if (i < len) {
            float r[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) r[e] = hv[j][e] + (v[j][e] * inv) * (w_offset + wv[j][e]);
            Quad<float>::store(h + base + i, r);
            if (copy != nullptr) Quad<TC>::store(copy + base + i, r);
        }
    }
}

// h [rows, len] float32; y [rows, len] or a stack [splits, rows, len] (y_dtype), or null; w [len] (w_dtype); copy [rows, len] (copy_dtype) or null.
extern "C" int spy_residual_norm(float* h, const void* y, int y_dtype, int splits, long long split_stride, const void* w, int w_dtype, float w_offset,
                                 void* copy, int copy_dtype, int rows, int len, float eps, cudaStream_t stream)
{
    if (rows <= 0) return 0;
    if (len <= 0) SPY_FAIL("residual_norm: row length %d must be positive", len);
    if (y != nullptr && (splits <= 0 || w == nullptr)) SPY_FAIL("residual_norm: a result to add needs its parts' count and the norm's weight");
    const size_t smem = (size_t)(len + 33) * sizeof(float);
    if (smem > 200 * 1024) SPY_FAIL("residual_norm: a row of %d does not fit a block's shared memory", len);
    if (y == nullptr) { y_dtype = SPY_F32; w_dtype = SPY_F32; }
    const bool aligned = (reinterpret_cast<uintptr_t>(h) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(copy) & 15) == 0 && (split_stride & 3) == 0;
    if (y != nullptr && len % 4 == 0 && len <= 16384 && aligned) {
        const int quads = len / 4;
        int nq = rows >= 4 * spy_sm_count() ? 4 : 1;            // many rows: fewer, fatter threads; few rows (decoding): the whole block on one row
        while (quads > nq * 1024) nq *= 2;
        int threads = ((quads + nq - 1) / nq + 31) / 32 * 32;
        SPY_DISPATCH_DTYPE(y_dtype, TY, {
            SPY_DISPATCH_DTYPE(w_dtype, TW, {
                SPY_DISPATCH_DTYPE(copy_dtype, TC, {
                    if (nq == 1) spy_launch(residual_norm_row_kernel<TY, TW, TC, 1, 1024>, dim3(rows), dim3(threads), 0, stream, h, (const TY*)y, splits, split_stride, (const TW*)w, w_offset, (TC*)copy, len, eps);
                    else if (nq == 2) spy_launch(residual_norm_row_kernel<TY, TW, TC, 2, 1024>, dim3(rows), dim3(threads), 0, stream, h, (const TY*)y, splits, split_stride, (const TW*)w, w_offset, (TC*)copy, len, eps);
                    else if (threads <= 256) spy_launch(residual_norm_row_kernel<TY, TW, TC, 4, 256>, dim3(rows), dim3(threads), 0, stream, h, (const TY*)y, splits, split_stride, (const TW*)w, w_offset, (TC*)copy, len, eps);
                    else spy_launch(residual_norm_row_kernel<TY, TW, TC, 4, 1024>, dim3(rows), dim3(threads), 0, stream, h, (const TY*)y, splits, split_stride, (const TW*)w, w_offset, (TC*)copy, len, eps);
                })
            })
        })
        SPY_CHECK_LAUNCH("residual_norm");
        return 0;
    }
    SPY_DISPATCH_DTYPE(y_dtype, TY, {
        SPY_DISPATCH_DTYPE(w_dtype, TW, {
            SPY_DISPATCH_DTYPE(copy_dtype, TC, {
                auto kernel = residual_norm_kernel<TY, TW, TC>;
                if (smem > 48 * 1024) SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                spy_launch(kernel, dim3(rows), dim3(256), smem, stream, h, (const TY*)y, splits, split_stride, (const TW*)w, w_offset, (TC*)copy, len, eps);
            })
        })
    })
    SPY_CHECK_LAUNCH("residual_norm");
    return 0;
}
