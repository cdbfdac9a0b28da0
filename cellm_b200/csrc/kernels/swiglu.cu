// SwiGLU gate: h[t, j] = g * sigmoid(g) * u with g = gu[t, j], u = gu[t, ff + j]
// (crates/cellm-model/src/lfm.rs:648-654; the two products W1 m and W3 m arrive
// side by side from one matrix product over the stacked weights). 32-bit math; gate and
// up may arrive in 32-bit under bfloat16 activations, so that the only rounding is that of h.
#include "common.cuh"

template <typename T, typename TI>
__global__ void swiglu_kernel(T* __restrict__ h, const TI* __restrict__ gu, int ff, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / ff;
    const int j = (int)(i - t * ff);
    const float g = to_float(gu[t * 2 * ff + j]);
    const float u = to_float(gu[t * 2 * ff + ff + j]);
    h[i] = from_float<T>(g * (1.0f / (1.0f + expf(-g))) * u);
}

CELLM_API int cellm_swiglu(void* h, const void* gu, int T, int ff, int dtype, int gu_dtype, cudaStream_t stream) {
    const size_t n = (size_t)T * ff;
    if (n == 0) return CELLM_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == CELLM_F32 && gu_dtype == CELLM_F32)
        CELLM_RUN((swiglu_kernel<float, float>), blocks, threads, 0, stream, (float*)h, (const float*)gu, ff, n);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_BF16)
        CELLM_RUN((swiglu_kernel<__nv_bfloat16, __nv_bfloat16>), blocks, threads, 0, stream, (__nv_bfloat16*)h, (const __nv_bfloat16*)gu, ff, n);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_F32)
        CELLM_RUN((swiglu_kernel<__nv_bfloat16, float>), blocks, threads, 0, stream, (__nv_bfloat16*)h, (const float*)gu, ff, n);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// The gated feed-forward's middle in its general form: h[t, j] = act(g + bg[j]) * (u + bu[j]) with g = gu[t, j],
// u = gu[t, ff + j]; act is silu (0) or the tanh form of gelu (1): 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
// The biases may be absent. 32-bit math.
template <typename T, typename TI, typename TW>
__global__ void gated_act_kernel(T* __restrict__ h, const TI* __restrict__ gu, long long ld, const TW* __restrict__ bg,
                                 const TW* __restrict__ bu, int ff, int act, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / ff;
    const int j = (int)(i - t * ff);
    float g = to_float(gu[t * ld + j]);
    float u = to_float(gu[t * ld + ff + j]);
    if (bg) g += to_float(bg[j]);
    if (bu) u += to_float(bu[j]);
    float a;
    if (act == 1) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else a = g * (1.0f / (1.0f + expf(-g)));
    h[i] = from_float<T>(a * u);
}

// The same, four neighbouring outputs a thread in 16-byte loads of 32-bit gate and up (ff a multiple of 4).
template <typename T, typename TW>
__global__ void gated_act_vec4_kernel(T* __restrict__ h, const float* __restrict__ gu, long long ld, const TW* __restrict__ bg,
                                      const TW* __restrict__ bu, int ff, int act, size_t n4) {
    pdl_trigger();
    pdl_wait();
    const size_t i4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i4 >= n4) return;
    const size_t i = i4 * 4;
    const size_t t = i / ff;
    const int j = (int)(i - t * ff);
    const float4 gq = *reinterpret_cast<const float4*>(gu + t * ld + j);
    const float4 uq = *reinterpret_cast<const float4*>(gu + t * ld + ff + j);
    float g[4] = {gq.x, gq.y, gq.z, gq.w}, u[4] = {uq.x, uq.y, uq.z, uq.w}, o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (bg) g[e] += to_float(bg[j + e]);
        if (bu) u[e] += to_float(bu[j + e]);
        const float a = act == 1 ? 0.5f * g[e] * (1.0f + tanhf(0.7978845608028654f * (g[e] + 0.044715f * g[e] * g[e] * g[e])))
                                 : g[e] * (1.0f / (1.0f + expf(-g[e])));
        o[e] = a * u[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) h[i + e] = from_float<T>(o[e]);
}

CELLM_API int cellm_gated_act(void* h, const void* gu, long long ld, const void* bg, const void* bu, int w_dtype, int T, int ff, int act,
                              int dtype, int gu_dtype, cudaStream_t stream) {
    const size_t n = (size_t)T * ff;
    if (n == 0) return CELLM_OK;
    if (act != 0 && act != 1) return CELLM_ERR_ARG;
    if (ld < 2LL * ff) return CELLM_ERR_SIZE;
    const int threads = 256;
    if (gu_dtype == CELLM_F32 && (ff & 3) == 0 && (ld & 3) == 0 && ((uintptr_t)gu & 15) == 0) {
        const size_t n4 = n / 4;
        const unsigned vblocks = (unsigned)((n4 + threads - 1) / threads);
#define VEC(TT, TW) CELLM_RUN((gated_act_vec4_kernel<TT, TW>), vblocks, threads, 0, stream, (TT*)h, (const float*)gu, ld, (const TW*)bg, (const TW*)bu, ff, act, n4)
        if (dtype == CELLM_F32 && w_dtype == CELLM_F32) VEC(float, float);
        else if (dtype == CELLM_F32 && w_dtype == CELLM_BF16) VEC(float, __nv_bfloat16);
        else if (dtype == CELLM_BF16 && w_dtype == CELLM_BF16) VEC(__nv_bfloat16, __nv_bfloat16);
        else if (dtype == CELLM_BF16 && w_dtype == CELLM_F32) VEC(__nv_bfloat16, float);
        else return CELLM_ERR_DTYPE;
#undef VEC
        return CELLM_OK;
    }
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
#define LAUNCH(TT, TI, TW) \
    CELLM_RUN((gated_act_kernel<TT, TI, TW>), blocks, threads, 0, stream, (TT*)h, (const TI*)gu, ld, (const TW*)bg, (const TW*)bu, ff, act, n)
    if (dtype == CELLM_F32 && gu_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float, float);
    else if (dtype == CELLM_F32 && gu_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, float, __nv_bfloat16);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, float, __nv_bfloat16);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float, float);
    else if (dtype == CELLM_BF16 && gu_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}

// out[t, i] = in[t, i] + b[i]: a product's 32-bit sums take their bias before they are rounded to the activations' type.
template <typename T, typename TW>
__global__ void bias_add_kernel(T* __restrict__ out, const float* __restrict__ in, const TW* __restrict__ b, int N, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = from_float<T>(in[i] + to_float(b[i % N]));
}

CELLM_API int cellm_bias_add(void* out, const float* in, const void* b, int w_dtype, int T, int N, int dtype, cudaStream_t stream) {
    const size_t n = (size_t)T * N;
    if (n == 0) return CELLM_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
#define LAUNCH(TT, TW) CELLM_RUN((bias_add_kernel<TT, TW>), blocks, 256, 0, stream, (TT*)out, in, (const TW*)b, N, n)
    if (dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float);
    else if (dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}
