// minGRU: a gated recurrence whose gates read only the current token.
//
//   z = sigmoid(pz + bz)      u = px + bx      c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//   S_t = (1 - z) S_(t-1) + z c               out_t = S_t * silu(pg)
//
// pz, px, pg arrive side by side from one product over the stacked matrices, [T, 3W]. The state S is one float per
// channel and request, kept in the request's slot between steps and zero at its start. Gates, candidate and state
// are 32-bit whatever the activations are. One thread per (request, channel) walks the request's tokens of this step in
// order, so the state after a token does not depend on how the sequence was cut into steps.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename TP, typename TA, typename TW>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(TA* __restrict__ out, const TP* __restrict__ proj, long long ld, const TW* __restrict__ bz,
                   const TW* __restrict__ bx, float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ slot_ids, const int* __restrict__ cu_seqlens, int W, int n_slots,
                   int* __restrict__ err) {
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= W) return;
    // the step's index arrays and the state are not the work of the kernel before this one
    const int slot = slot_ids[b];
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    if (slot < 0 || slot >= n_slots) {
        if (c == 0) atomicOr(err, CELLM_DEV_BAD_SLOT);
        return;
    }
    const float zb = bz ? to_float(bz[c]) : 0.f, xb = bx ? to_float(bx[c]) : 0.f;
    float S = state[(size_t)slot * slot_stride + c];
    pdl_wait();
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        const TP* row = proj + (size_t)t * ld;
        const float z = sigmoid_f(to_float(row[c]) + zb);
        const float u = to_float(row[W + c]) + xb;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        const float g = to_float(row[2 * W + c]);
        S = (1.0f - z) * S + z * cand;
        out[(size_t)t * W + c] = from_float<TA>(S * (g * sigmoid_f(g)));
    }
    state[(size_t)slot * slot_stride + c] = S;
}

// Long portions: the recurrence is linear in S (S_t = a_t S_(t-1) + b_t with a = 1 - z, b = z c), so a portion is cut
// into MG_SEGS runs of tokens that are walked side by side. A block is MG_CH channels times MG_SEGS runs (a half warp reads 16 neighbouring channels of a token). Each thread
// first walks its run from zero and keeps (product of a, end value); the run's true start follows from the runs before
// it (at most MG_SEGS - 1 steps of S <- A S + B, from the state the request brought); then the run is walked again from
// that start and the outputs are written. The sums differ from the token-by-token walk only in rounding.
#define MG_SEGS 64
#define MG_CH 16
template <typename TP, typename TA, typename TW>
__global__ void __launch_bounds__(MG_CH * MG_SEGS)
mingru_chunked_kernel(TA* __restrict__ out, const TP* __restrict__ proj, long long ld, const TW* __restrict__ bz,
                      const TW* __restrict__ bx, float* __restrict__ state, long long slot_stride,
                      const int* __restrict__ slot_ids, const int* __restrict__ cu_seqlens, int W, int n_slots,
                      int* __restrict__ err) {
    __shared__ float prod_s[MG_SEGS][MG_CH + 1], end_s[MG_SEGS][MG_CH + 1];
    pdl_trigger();
    const int lane = threadIdx.x, seg = threadIdx.y;
    const int c = blockIdx.x * MG_CH + lane;
    const int b = blockIdx.y;
    const int slot = slot_ids[b];
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const bool slot_ok = slot >= 0 && slot < n_slots;
    if (!slot_ok && lane == 0 && seg == 0 && blockIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_SLOT);
    const bool on = c < W && slot_ok;
    const int per = (t1 - t0 + MG_SEGS - 1) / MG_SEGS;
    const int lo = min(t1, t0 + seg * per), hi = min(t1, lo + per);
    const float zb = (on && bz) ? to_float(bz[c]) : 0.f, xb = (on && bx) ? to_float(bx[c]) : 0.f;
    const float S0 = on ? state[(size_t)slot * slot_stride + c] : 0.f;
    pdl_wait();
    float A = 1.f, E = 0.f;
    if (on) {
#pragma unroll 4
        for (int t = lo; t < hi; ++t) {
            const TP* row = proj + (size_t)t * ld;
            const float z = sigmoid_f(to_float(row[c]) + zb);
            const float u = to_float(row[W + c]) + xb;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            A *= 1.0f - z;
            E = (1.0f - z) * E + z * cand;
        }
    }
    prod_s[seg][lane] = A;
    end_s[seg][lane] = E;
    __syncthreads();
    float S = S0;
    for (int k = 0; k < seg; ++k) S = prod_s[k][lane] * S + end_s[k][lane];
    if (on) {
#pragma unroll 4
        for (int t = lo; t < hi; ++t) {
            const TP* row = proj + (size_t)t * ld;
            const float z = sigmoid_f(to_float(row[c]) + zb);
            const float u = to_float(row[W + c]) + xb;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            const float g = to_float(row[2 * W + c]);
            S = (1.0f - z) * S + z * cand;
            out[(size_t)t * W + c] = from_float<TA>(S * (g * sigmoid_f(g)));
        }
        if (seg == MG_SEGS - 1) state[(size_t)slot * slot_stride + c] = S;
    }
}

// out: [T, W] activations; proj: [T, ld] = [pz | px | pg] (32-bit, or the activations' type); bz, bx: [W] or null;
// state: [slots, slot_stride] float, read and updated in place. max_q_len: the longest portion of the step (0: unknown).
CELLM_API int cellm_mingru_scan(void* out, const void* proj, long long ld, int proj_dtype, const void* bz, const void* bx,
                                int w_dtype, float* state, long long slot_stride, const int* slot_ids, const int* cu_seqlens,
                                int T, int B, int W, int n_slots, int max_q_len, int act_dtype, int* err, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return CELLM_OK;
    if (W <= 0 || ld < 3LL * W) return CELLM_ERR_SIZE;
    if (!state || !proj || !out) return CELLM_ERR_ARG;
    // long portions under 16-bit activations walk their tokens in runs side by side (max_q_len: the longest portion if the
    // host knows it, else 0); 32-bit activations always take the token-by-token walk, whose sums do not depend on the cut
    if (act_dtype == CELLM_BF16 && max_q_len >= 2 * MG_SEGS) {
        const dim3 cgrid((unsigned)((W + MG_CH - 1) / MG_CH), (unsigned)B), cblock(MG_CH, MG_SEGS);
#define CHUNKED(TP, TW)                                                                                                 \
        CELLM_RUN((mingru_chunked_kernel<TP, __nv_bfloat16, TW>), cgrid, cblock, 0, stream, (__nv_bfloat16*)out, (const TP*)proj, ld, \
                  (const TW*)bz, (const TW*)bx, state, slot_stride, slot_ids, cu_seqlens, W, n_slots, err)
        if (proj_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) CHUNKED(__nv_bfloat16, __nv_bfloat16);
        else if (proj_dtype == CELLM_BF16 && w_dtype == CELLM_F32) CHUNKED(__nv_bfloat16, float);
        else if (w_dtype == CELLM_BF16) CHUNKED(float, __nv_bfloat16);
        else if (w_dtype == CELLM_F32) CHUNKED(float, float);
        else return CELLM_ERR_DTYPE;
#undef CHUNKED
        return CELLM_OK;
    }
    const dim3 grid((unsigned)((W + 127) / 128), (unsigned)B);
#define LAUNCH(TP, TA, TW)                                                                                              \
    CELLM_RUN((mingru_scan_kernel<TP, TA, TW>), grid, 128, 0, stream, (TA*)out, (const TP*)proj, ld, (const TW*)bz, (const TW*)bx, \
              state, slot_stride, slot_ids, cu_seqlens, W, n_slots, err)
    if (act_dtype == CELLM_F32 && proj_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, float, float);
    else if (act_dtype == CELLM_F32 && proj_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_F32 && w_dtype == CELLM_BF16) LAUNCH(float, __nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_F32 && w_dtype == CELLM_F32) LAUNCH(float, __nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_BF16 && w_dtype == CELLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && proj_dtype == CELLM_BF16 && w_dtype == CELLM_F32) LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
    else return CELLM_ERR_DTYPE;
#undef LAUNCH
    return CELLM_OK;
}
