// The norm of a layer that normalises AFTER the sum: the stream is replaced by
//
//   h <- rms(alpha * h + a + s * b) * w        rms(x) = x / sqrt(mean(x^2) + eps)
//
// with a and b what the sub-layer produced (each float32 [T, E], or partial sums [parts, T, E] that are added in
// order; either may be absent) and s an optional factor per row for b (a gate of one number per token).  The sum,
// the mean of squares and the product are 32-bit; the new stream is written back in float32 and, for the matrix
// products that read it next, in the compute dtype.
//
// Without w only the sum is written back.  One block per row; the row waits in shared memory between the two passes.
#include "common.cuh"

namespace air {

template <typename TW, typename TO>
__global__ void __launch_bounds__(1024)
post_norm_kernel(float* __restrict__ h, float alpha, const float* __restrict__ a, int a_parts,
                 const float* __restrict__ b, int b_parts, const float* __restrict__ b_row_scale, size_t part_stride,
                 const TW* __restrict__ w, TO* __restrict__ out, int E, float eps) {
    extern __shared__ float xrow[];
    __shared__ float scratch[32];
    pdl_enter(TR_POST_NORM);
    const size_t src = (size_t)blockIdx.x * E;
    const float sb = b_row_scale ? b_row_scale[blockIdx.x] : 1.f;
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float x = alpha * h[src + i];
        if (a) {
            float t = a[src + i];
            for (int p = 1; p < a_parts; ++p) t += a[p * part_stride + src + i];
            x += t;
        }
        if (b) {
            float t = b[src + i];
            for (int p = 1; p < b_parts; ++p) t += b[p * part_stride + src + i];
            x += sb * t;
        }
        xrow[i] = x;
        ss += x * x;
    }
    if (!w) {      // only the sum is wanted
        for (int i = threadIdx.x; i < E; i += blockDim.x) h[src + i] = xrow[i];
        return;
    }
    const float total = block_sum(ss, scratch);
    const float scale = 1.f / sqrtf(total / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float y = xrow[i] * scale * to_float(w[i]);
        h[src + i] = y;
        if (out) out[src + i] = from_float<TO>(y);
    }
}

}  // namespace air

AIR_API int air_post_norm(float* h, float alpha, const float* a, int a_parts, const float* b, int b_parts,
                          const float* b_row_scale, long long part_stride, const void* w, int w_dtype, void* out,
                          int out_dtype, int T, int E, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    int threads = E >= 2048 ? 512 : (E >= 512 ? 256 : 128);
    if (T <= 256) threads = E / 2 >= 1024 ? 1024 : (E / 2 > threads ? (E / 2 + 31) / 32 * 32 : threads);
    const size_t smem = sizeof(float) * (size_t)E;
    if (smem > 200 * 1024) return AIR_ERR_BAD_ARGUMENT;
    if (!w) w_dtype = AIR_F32;
    AIR_DISPATCH(w_dtype, TW, AIR_DISPATCH(out_dtype, TO, {
        auto kernel = air::post_norm_kernel<TW, TO>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return air::launch(kernel, T, threads, smem, stream, h, alpha, a, a_parts, b, b_parts, b_row_scale,
                           (size_t)part_stride, (const TW*)w, (TO*)out, E, eps);
    }));
    return 0;
}

AIR_API int air_trace_set_post_norm(unsigned long long* buffer) { return air::set_trace_here(buffer); }
