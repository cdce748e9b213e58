// Backward of the epilogue that the aggregation kernels fuse (row scale, bias, activation): one streaming pass
//   grad_agg[r,d] = grad_y[r,d] * act'(y[r,d]) * row_scale[r]
// where the reference's layers run two or three element-wise torch kernels.  HBM-bound: 12 bytes per element
// (two reads, one write); 128-bit accesses when the row width allows, grid sized to a few waves of the SMs.
#include "common.cuh"

namespace yitu {

__device__ __forceinline__ float act_grad(float y, int act) {
    if (act == YITU_ACT_RELU) return y > 0.0f ? 1.0f : 0.0f;
    if (act == YITU_ACT_ELU) return y > 0.0f ? 1.0f : y + 1.0f;
    return 1.0f;
}

template <int VEC>
__global__ void __launch_bounds__(256)
epilogue_grad_kernel(int64_t n_rows, int64_t D, int act, const float *y, const float *gy, const float *row_scale,
                     float *out) {
    const int64_t per_row = D / VEC;
    const int64_t total = n_rows * per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const float s = row_scale ? __ldg(row_scale + i / per_row) : 1.0f;
        if constexpr (VEC == 4) {
            const float4 g = __ldcs(reinterpret_cast<const float4 *>(gy) + i);
            float4 d = make_float4(s, s, s, s);
            if (act) {
                const float4 v = __ldcs(reinterpret_cast<const float4 *>(y) + i);
                d.x *= act_grad(v.x, act); d.y *= act_grad(v.y, act); d.z *= act_grad(v.z, act); d.w *= act_grad(v.w, act);
            }
            __stcs(reinterpret_cast<float4 *>(out) + i, make_float4(g.x * d.x, g.y * d.y, g.z * d.z, g.w * d.w));
        } else {
            const float d = act ? act_grad(__ldcs(y + i), act) : 1.0f;
            __stcs(out + i, __ldcs(gy + i) * d * s);
        }
    }
}

}  // namespace yitu

using namespace yitu;

extern "C" int yitu_epilogue_grad_f32(int64_t n_rows, int64_t n_feats, int32_t activation, const float *y,
                                      const float *grad_y, const float *row_scale, float *grad_agg,
                                      yitu_stream_t stream) {
    YITU_REQUIRE(n_rows >= 0 && n_feats >= 1, YITU_ERR_INVALID_ARG, "bad shape (%lld x %lld)", (long long)n_rows,
                 (long long)n_feats);
    YITU_REQUIRE(activation >= YITU_ACT_NONE && activation <= YITU_ACT_ELU, YITU_ERR_INVALID_ARG,
                 "unknown activation %d", activation);
    if (n_rows == 0) return YITU_OK;
    YITU_REQUIRE(grad_y && grad_agg && (activation == YITU_ACT_NONE || y), YITU_ERR_INVALID_ARG, "NULL tensor");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool vec = n_feats % 4 == 0 && aligned16(grad_y) && aligned16(grad_agg) && (y == nullptr || aligned16(y));
    const int64_t total = n_rows * (vec ? n_feats / 4 : n_feats);
    const int64_t want = (total + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
    if (vec) epilogue_grad_kernel<4><<<blocks, 256, 0, st>>>(n_rows, n_feats, activation, y, grad_y, row_scale, grad_agg);
    else epilogue_grad_kernel<1><<<blocks, 256, 0, st>>>(n_rows, n_feats, activation, y, grad_y, row_scale, grad_agg);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}
