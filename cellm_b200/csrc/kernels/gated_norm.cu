// A sublayer's result joins the residual stream through a gate and a norm:
//
//   v[t]  = m[t] * sigmoid(g[t] + b)          (the gate is optional: without it v = m)
//   x[t] += v[t] / rms_per_group(v[t]) * w    (the row in `groups` equal consecutive parts, each divided by its own
//                                              sqrt(mean(part^2) + eps))
//   y[t]  = x[t] in the activations' element type (optional: what the next sublayer's products read)
//
// m is a mixer's or feed-forward's output, g the gate's pre-activation (a product over the sublayer's input). Gate,
// norm and sum are 32-bit; the stream x is 32-bit in every mode. One block per row; the order of every sum depends on
// the row length and the block size only.
#include "common.cuh"

template <typename TA, typename TW>
__global__ void gated_norm_add_kernel(float* __restrict__ x, const TA* __restrict__ m, const TA* __restrict__ gate,
                                      const TW* __restrict__ gate_bias, const TW* __restrict__ w, TA* __restrict__ y,
                                      int H, int groups, float eps) {
    extern __shared__ float vals[];      // [H]
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * H;
    const int Hg = H / groups;
    for (int g = 0; g < groups; ++g) {
        const int lo = g * Hg, hi = lo + Hg;
        float ss = 0.f;
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            float v = to_float(m[row + i]);
            if (gate) {
                float z = to_float(gate[row + i]);
                if (gate_bias) z += to_float(gate_bias[i]);
                v *= 1.0f / (1.0f + expf(-z));
            }
            vals[i] = v;
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)Hg + eps);
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float xv = x[row + i] + vals[i] * inv * to_float(w[i]);
            x[row + i] = xv;
            if (y) y[row + i] = from_float<TA>(xv);
        }
    }
}

// x: [T, H] float, updated in place; m, gate: [T, H] of the activations' type (gate may be null); gate_bias, w: [H] of the
// weights' type (gate_bias may be null); y: [T, H] of the activations' type or null.
CELLM_API int cellm_gated_norm_add(float* x, const void* m, const void* gate, const void* gate_bias, const void* w, int w_dtype,
                                   void* y, int T, int H, int groups, float eps, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (groups < 1 || H % groups || H <= 0) return CELLM_ERR_SIZE;
    if (!x || !m || !w) return CELLM_ERR_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    const int per = H / groups;
    const int threads = per >= 2048 ? 512 : (per >= 512 ? 256 : 128);
#define LAUNCH(TA, TW)                                                                                                 \
    do {                                                                                                               \
        if (smem > 48 * 1024) cudaFuncSetAttribute(gated_norm_add_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        CELLM_RUN((gated_norm_add_kernel<TA, TW>), T, threads, smem, stream, x, (const TA*)m, (const TA*)gate,          \
                  (const TW*)gate_bias, (const TW*)w, (TA*)y, H, groups, eps);                                          \
    } while (0)
    if (act_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float);
    else if (act_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}

// y = x in the activations' element type: what a sublayer that reads the stream itself takes its products from.
template <typename TA>
__global__ void stream_cast_kernel(TA* __restrict__ y, const float* __restrict__ x, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = from_float<TA>(x[i]);
}

CELLM_API int cellm_stream_cast(void* y, const float* x, long long n, int act_dtype, cudaStream_t stream) {
    if (n <= 0) return CELLM_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_dtype == CELLM_F32) CELLM_RUN(stream_cast_kernel<float>, blocks, 256, 0, stream, (float*)y, x, (size_t)n);
    else if (act_dtype == CELLM_BF16) CELLM_RUN(stream_cast_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)y, x, (size_t)n);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}
