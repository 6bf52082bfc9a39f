// The residual sum of a block whose norm sits on the sublayer's OUTPUT:  h += rms_norm(y) * w,  h the 32-bit residual stream.
//   v   = y[row], itself possibly a sum of split-K partial products            32-bit sums
//   h[row] += v * (1 / sqrt(mean(v^2) + eps)) * w                              32-bit statistics; w as stored or as (offset + w)
//   copy[row] = h[row] in the activations' type                                what the next sublayer's products read (optional)
// With y absent the kernel only makes the copy (the embedding's rows for the first sublayer).
// One block a row; the row waits in shared memory between the two passes.
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
