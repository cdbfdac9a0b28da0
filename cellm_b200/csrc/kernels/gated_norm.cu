// A sublayer's result joins the residual stream through a gate and a norm:
//
//   v[t]  = (m[t] + c) * sigmoid(g[t] + b)    (the gate is optional: without it v = m + c; so is c, a bias that the
//                                              product behind m has not taken yet)
//   x[t] += v[t] / rms_per_group(v[t]) * w    (the row in `groups` equal consecutive parts, each divided by its own
//                                              sqrt(mean(part^2) + eps))
//   y[t]  = x[t] in the activations' element type (optional: what the next sublayer's products read)
//
// m is a mixer's or feed-forward's output, g the gate's pre-activation (a product over the sublayer's input; it may
// lie in a wider matrix, behind the columns of the sublayer's own first product, and be 32-bit there). Gate,
// norm and sum are 32-bit; the stream x is 32-bit in every mode. One block per row; the order of every sum depends on
// the row length and the block size only.
#include "common.cuh"

template <typename TA, typename TW, typename TG>
__global__ void gated_norm_add_kernel(float* __restrict__ x, const TA* __restrict__ m, const TW* __restrict__ m_bias, const TG* __restrict__ gate,
                                      long long gld, const TW* __restrict__ gate_bias, const TW* __restrict__ w, TA* __restrict__ y,
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
            if (m_bias) v += to_float(m_bias[i]);
            if (gate) {
                float z = to_float(gate[(size_t)blockIdx.x * gld + i]);
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

// The same for bfloat16 activations and weights when a group is a multiple of 8 values and at most 8 * 1024: one block
// per (row, group), every thread keeps its 8 values in registers, each element is read once and written once in
// 16-byte pieces. The group's sum is taken in an order that depends on its length only.
template <typename TG>
__global__ void gated_norm_add_vec8_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ m,
                                           const __nv_bfloat16* __restrict__ m_bias,
                                           const TG* __restrict__ gate, long long gld, const __nv_bfloat16* __restrict__ gate_bias,
                                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int H, int Hg,
                                           float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    const int i0 = threadIdx.x * 8;
    const bool on = i0 < Hg;
    const int col = blockIdx.y * Hg + i0;
    const size_t at = (size_t)blockIdx.x * H + col;
    float wv[8], bv[8], cv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] = bv[j] = cv[j] = 0.f;
    if (on) {                                   // weights and bias are not the work of the kernel before this one
        const uint4 wq = *reinterpret_cast<const uint4*>(w + col);
        const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wq);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(wp[j]); wv[2 * j] = f.x; wv[2 * j + 1] = f.y; }
        if (m_bias) {
            const uint4 cq = *reinterpret_cast<const uint4*>(m_bias + col);
            const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&cq);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(cp[j]); cv[2 * j] = f.x; cv[2 * j + 1] = f.y; }
        }
        if (gate_bias) {
            const uint4 bq = *reinterpret_cast<const uint4*>(gate_bias + col);
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bq);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(bp[j]); bv[2 * j] = f.x; bv[2 * j + 1] = f.y; }
        }
    }
    pdl_wait();
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (on) {
        const uint4 mq = *reinterpret_cast<const uint4*>(m + at);
        const __nv_bfloat162* mp = reinterpret_cast<const __nv_bfloat162*>(&mq);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(mp[j]); v[2 * j] = f.x + cv[2 * j]; v[2 * j + 1] = f.y + cv[2 * j + 1]; }
        if (gate) {
            float z[8];
            const TG* gr = gate + (size_t)blockIdx.x * gld + col;
            if constexpr (sizeof(TG) == 4) {
                const float4 g0 = *reinterpret_cast<const float4*>(gr), g1 = *reinterpret_cast<const float4*>(gr + 4);
                z[0] = g0.x; z[1] = g0.y; z[2] = g0.z; z[3] = g0.w; z[4] = g1.x; z[5] = g1.y; z[6] = g1.z; z[7] = g1.w;
            } else {
                const uint4 gq = *reinterpret_cast<const uint4*>(gr);
                const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gq);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(gp[j]); z[2 * j] = f.x; z[2 * j + 1] = f.y; }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= 1.0f / (1.0f + expf(-(z[j] + bv[j])));
        }
    }
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;          // the stream's values travel while the group's sum is taken
    if (on) {
        a = *reinterpret_cast<const float4*>(x + at);
        b = *reinterpret_cast<const float4*>(x + at + 4);
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)Hg + eps);
    if (on) {
        float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) xv[j] += v[j] * inv * wv[j];
        *reinterpret_cast<float4*>(x + at) = make_float4(xv[0], xv[1], xv[2], xv[3]);
        *reinterpret_cast<float4*>(x + at + 4) = make_float4(xv[4], xv[5], xv[6], xv[7]);
        if (y) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 pk = __floats2bfloat162_rn(xv[2 * j], xv[2 * j + 1]);
                o[j] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(y + at) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// x: [T, H] float, updated in place; m: [T, H] of the activations' type; gate: [T, H] at row pitch gate_ld, of the activations'
// type or 32-bit (gate_dtype), or null; m_bias, gate_bias, w: [H] of the weights' type (the biases may be null); y: [T, H] of the activations' type or null.
CELLM_API int cellm_gated_norm_add(float* x, const void* m, const void* m_bias, const void* gate, long long gate_ld, int gate_dtype,
                                   const void* gate_bias, const void* w, int w_dtype,
                                   void* y, int T, int H, int groups, float eps, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (groups < 1 || H % groups || H <= 0) return CELLM_ERR_SIZE;
    if (!x || !m || !w) return CELLM_ERR_ARG;
    if (gate && (gate_ld < H || (gate_dtype != CELLM_F32 && gate_dtype != act_dtype))) return CELLM_ERR_ARG;
    const bool gate32 = gate && gate_dtype == CELLM_F32 && act_dtype != CELLM_F32;
    const int Hg = H / groups;
    if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16 && (Hg & 7) == 0 && Hg <= 8192 &&
        (((uintptr_t)x | (uintptr_t)m | (uintptr_t)m_bias | (uintptr_t)gate | (uintptr_t)gate_bias | (uintptr_t)w | (uintptr_t)y) & 15) == 0 &&
        (gate_ld & 7) == 0) {
        const int vthreads = ((Hg / 8 + 31) / 32) * 32;
        if (gate32)
            CELLM_RUN(gated_norm_add_vec8_kernel<float>, dim3((unsigned)T, (unsigned)groups), vthreads, 0, stream, x, (const __nv_bfloat16*)m,
                      (const __nv_bfloat16*)m_bias, (const float*)gate, gate_ld, (const __nv_bfloat16*)gate_bias, (const __nv_bfloat16*)w,
                      (__nv_bfloat16*)y, H, Hg, eps);
        else
            CELLM_RUN(gated_norm_add_vec8_kernel<__nv_bfloat16>, dim3((unsigned)T, (unsigned)groups), vthreads, 0, stream, x,
                      (const __nv_bfloat16*)m, (const __nv_bfloat16*)m_bias, (const __nv_bfloat16*)gate, gate_ld,
                      (const __nv_bfloat16*)gate_bias, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, Hg, eps);
        return CELLM_OK;
    }
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    const int per = H / groups;
    const int threads = per >= 2048 ? 512 : (per >= 512 ? 256 : 128);
#define LAUNCH(TA, TW, TG)                                                                                             \
    do {                                                                                                               \
        if (smem > 48 * 1024) cudaFuncSetAttribute(gated_norm_add_kernel<TA, TW, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        CELLM_RUN((gated_norm_add_kernel<TA, TW, TG>), T, threads, smem, stream, x, (const TA*)m, (const TW*)m_bias, (const TG*)gate, gate_ld, \
                  (const TW*)gate_bias, (const TW*)w, (TA*)y, H, groups, eps);                                          \
    } while (0)
    if (act_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float, float);
    else if (act_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_F32 && gate32) LAUNCH(__nv_bfloat16, float, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16 && gate32) LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
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
