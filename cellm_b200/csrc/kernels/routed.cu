// Routed feed-forward ("mixture of experts"): the router with its choice of experts, and the experts' two
// products in the form that serves few tokens and the 32-bit path (a token's chosen experts are walked row by
// row; every weight row a token needs is read once for it).
//
//   z = R h (32-bit sums);  s = sigmoid(z);  c = s + correction          (c chooses, s weighs)
//   experts lie in `n_groups` equal runs of neighbours; a run's score is the sum of its two largest c (its
//   only c for runs of one); only experts of the `keep` best runs can be chosen (the others count as -inf)
//   the `top` experts with the largest c are chosen; their weights are s / (sum of the chosen s + 1e-20) * scale
//   out = sum_k weight_k * D_k act(U_k h)  [+ sigmoid(g . h) * shared(h)]
//
// Ties go to the lower index. The chosen experts are listed by descending c, and every sum runs in an order
// that depends on the sizes alone, so a token's result does not depend on what else is in the batch.
#include "common.cuh"

#define ROUTE_THREADS 512

// A lane's share of the dot product of a weight row with a vector held as floats: pieces of 16 bytes where the
// row allows it (`vec`), else element by element.
template <typename TW>
__device__ __forceinline__ float lane_dot(const TW* __restrict__ w, const float* __restrict__ v, int n, int lane, bool vec);
template <>
__device__ __forceinline__ float lane_dot<float>(const float* __restrict__ w, const float* __restrict__ v, int n, int lane, bool vec) {
    float a = 0.f;
    if (vec) {
#pragma unroll 4
        for (int i = lane * 4; i < n; i += 128) {
            const float4 x = *reinterpret_cast<const float4*>(w + i);
            const float4 y = *reinterpret_cast<const float4*>(v + i);
            a += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
        }
    } else {
        for (int i = lane; i < n; i += 32) a += w[i] * v[i];
    }
    return a;
}
template <>
__device__ __forceinline__ float lane_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ v, int n, int lane,
                                                        bool vec) {
    float a = 0.f;
    if (vec) {
#pragma unroll 4
        for (int i = lane * 8; i < n; i += 256) {
            const uint4 x = *reinterpret_cast<const uint4*>(w + i);
            const float4 y0 = *reinterpret_cast<const float4*>(v + i), y1 = *reinterpret_cast<const float4*>(v + i + 4);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&x);
            const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]), f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
            a += f0.x * y0.x + f0.y * y0.y + f1.x * y0.z + f1.y * y0.w + f2.x * y1.x + f2.y * y1.y + f3.x * y1.z + f3.y * y1.w;
        }
    } else {
        for (int i = lane; i < n; i += 32) a += __bfloat162float(w[i]) * v[i];
    }
    return a;
}
template <typename TW> __device__ __forceinline__ bool rows_vectorise(const TW* base, long long ld, int n) {
    constexpr int per = 16 / (int)sizeof(TW);
    return (n % per) == 0 && (ld % per) == 0 && (((uintptr_t)base) & 15) == 0;
}

// ---- the router ----------------------------------------------------------------------------------------------------
// One block takes ROUTE_TPB tokens (8, or 1 where eight rows of the input do not fit shared memory): their inputs lie in shared memory, a warp forms one router row's sums for all of
// them at once, then a warp a token chooses.
template <int ROUTE_TPB, typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_kernel(int* __restrict__ idx, float* __restrict__ wts, float* __restrict__ gate_out, const TA* __restrict__ y, long long ldy,
             const TW* __restrict__ router, const TC* __restrict__ correction, int T, int H, int E, int top, int n_groups, int keep,
             float scale, int has_gate) {
    extern __shared__ __align__(16) float smem[];
    float* hs = smem;                               // [TPB][H]
    float* sc = hs + (size_t)ROUTE_TPB * H;         // [TPB][E + 1]: logits, then s
    float* ch = sc + ROUTE_TPB * (E + 1);           // [TPB][E]: choice scores
    float* gs = ch + ROUTE_TPB * E;                 // [TPB][n_groups]: scores of the runs
    float* kf = gs + ROUTE_TPB * n_groups;          // [TPB][n_groups]: 1 = the run is kept
    float* sel = kf + ROUTE_TPB * n_groups;         // [TPB][top]: s of the chosen, by rank
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = ROUTE_THREADS / 32;
    const int t0 = blockIdx.x * ROUTE_TPB, nt = min(ROUTE_TPB, T - t0);
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < ROUTE_TPB * H; i += ROUTE_THREADS) {
        const int j = i / H, c = i - j * H;
        hs[i] = j < nt ? to_float(y[(size_t)(t0 + j) * ldy + c]) : 0.f;
    }
    __syncthreads();
    const int rows = E + (has_gate ? 1 : 0);
    const bool vec = rows_vectorise(router, H, H);
    constexpr int PER = 16 / (int)sizeof(TW);       // elements in a 16-byte piece of a router row
    for (int r = warp; r < rows; r += nwarps) {
        float acc[ROUTE_TPB];
#pragma unroll
        for (int j = 0; j < ROUTE_TPB; ++j) acc[j] = 0.f;
        const TW* wr = router + (size_t)r * H;
        if (vec) {
            for (int i = lane * PER; i < H; i += 32 * PER) {
                float w[PER];
                const uint4 x = *reinterpret_cast<const uint4*>(wr + i);
                const TW* xp = reinterpret_cast<const TW*>(&x);
#pragma unroll
                for (int k = 0; k < PER; ++k) w[k] = to_float(xp[k]);
#pragma unroll
                for (int j = 0; j < ROUTE_TPB; ++j) {
                    if (j < nt) {
#pragma unroll
                        for (int k = 0; k < PER; k += 4) {
                            const float4 y = *reinterpret_cast<const float4*>(hs + j * H + i + k);
                            acc[j] += w[k] * y.x + w[k + 1] * y.y + w[k + 2] * y.z + w[k + 3] * y.w;
                        }
                    }
                }
            }
        } else {
            for (int i = lane; i < H; i += 32) {
                const float w = to_float(wr[i]);
#pragma unroll
                for (int j = 0; j < ROUTE_TPB; ++j) acc[j] += w * hs[j * H + i];
            }
        }
#pragma unroll
        for (int j = 0; j < ROUTE_TPB; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0) sc[j * (E + 1) + r] = v;
        }
    }
    __syncthreads();
    const int gsz = E / n_groups;
    for (int j = warp; j < nt; j += nwarps) {
        const int t = t0 + j;
        float* z = sc + j * (E + 1);
        float* c = ch + j * E;
        float* g = gs + j * n_groups;
        float* k = kf + j * n_groups;
        float* chosen = sel + j * top;
        for (int e = lane; e < E; e += 32) {
            const float s = 1.f / (1.f + expf(-z[e]));
            z[e] = s;
            c[e] = s + to_float(correction[e]);
        }
        if (has_gate && lane == 0) gate_out[t] = 1.f / (1.f + expf(-z[E]));
        __syncwarp();
        if (n_groups > 1) {
            for (int gi = lane; gi < n_groups; gi += 32) {
                float m1 = -INFINITY, m2 = -INFINITY;
                for (int e = gi * gsz; e < (gi + 1) * gsz; ++e) {
                    const float v = c[e];
                    if (v > m1) { m2 = m1; m1 = v; }
                    else if (v > m2) m2 = v;
                }
                g[gi] = gsz >= 2 ? m1 + m2 : m1;
            }
            __syncwarp();
            for (int gi = lane; gi < n_groups; gi += 32) {
                int rank = 0;
                const float mine = g[gi];
                for (int gj = 0; gj < n_groups; ++gj) rank += (g[gj] > mine || (g[gj] == mine && gj < gi)) ? 1 : 0;
                k[gi] = rank < keep ? 1.f : 0.f;
            }
            __syncwarp();
            for (int e = lane; e < E; e += 32)
                if (k[e / gsz] == 0.f) c[e] = -INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) {
            int rank = 0;
            const float mine = c[e];
            for (int f = 0; f < E; ++f) rank += (c[f] > mine || (c[f] == mine && f < e)) ? 1 : 0;
            if (rank < top) {
                idx[(size_t)t * top + rank] = e;
                chosen[rank] = z[e];
            }
        }
        __syncwarp();
        float sum = 0.f;
        for (int r = 0; r < top; ++r) sum += chosen[r];
        for (int r = lane; r < top; r += 32) wts[(size_t)t * top + r] = chosen[r] / (sum + 1e-20f) * scale;
    }
}

// y: [T, H] (row pitch ldy); router: [E (+1), H], row E the shared expert's gate when has_gate; correction: [E].
// idx: [T, top] int, wts: [T, top] float, gate_out: [T] float (sigmoid of the gate row's sum).
CELLM_API int cellm_route(int* idx, float* wts, float* gate_out, const void* y, long long ldy, const void* router, int w_dtype,
                          const void* correction, int c_dtype, int T, int H, int E, int top, int n_groups, int keep, float scale,
                          int has_gate, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (E < 1 || top < 1 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups || H < 1) return CELLM_ERR_SIZE;
    if (has_gate && !gate_out) return CELLM_ERR_ARG;
    if (w_dtype != act_dtype) return CELLM_ERR_DTYPE;
    const size_t per_token = ((size_t)H + 2 * E + 1 + 2 * n_groups + top) * sizeof(float);
    const int tpb = 8 * per_token <= 200 * 1024 ? 8 : 1;
    const size_t smem = tpb * per_token;
    if (smem > 200 * 1024) return CELLM_ERR_SIZE;
    const unsigned blocks = (unsigned)((T + tpb - 1) / tpb);
#define GO2(TPB, TA, TC)                                                                                                    \
    do {                                                                                                                    \
        static size_t configured = 0;                                                                                       \
        if (smem > 48 * 1024 && smem > configured) {                                                                        \
            const cudaError_t e = cudaFuncSetAttribute(route_kernel<TPB, TA, TA, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e;                                                                            \
            configured = 200 * 1024;                                                                                        \
        }                                                                                                                   \
        CELLM_RUN((route_kernel<TPB, TA, TA, TC>), blocks, ROUTE_THREADS, smem, stream, idx, wts, gate_out, (const TA*)y, ldy, \
                  (const TA*)router, (const TC*)correction, T, H, E, top, n_groups, keep, scale, has_gate);                 \
    } while (0)
#define GO(TA, TC)                          \
    do {                                    \
        if (tpb == 8) GO2(8, TA, TC);       \
        else GO2(1, TA, TC);                \
    } while (0)
    if (act_dtype == CELLM_F32 && c_dtype == CELLM_F32) GO(float, float);
    else if (act_dtype == CELLM_F32 && c_dtype == CELLM_BF16) GO(float, __nv_bfloat16);
    else if (act_dtype == CELLM_BF16 && c_dtype == CELLM_F32) GO(__nv_bfloat16, float);
    else if (act_dtype == CELLM_BF16 && c_dtype == CELLM_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef GO2
#undef GO
    return CELLM_OK;
}

// ---- the experts, row by row ----------------------------------------------------------------------------------------
#define EXPERT_THREADS 128
#define EXPERT_ROWS 4           // output rows a block forms: one a warp

// mid[t * top + k, :] = act(U_e y[t]) for e = idx[t, k]; up: [E * ff, H]. Blocks with blockIdx.x >= T * top take the shared
// expert: smid[t, :] = act(U_s y[t]), U_s: [sff, H].
template <typename TA>
__global__ void __launch_bounds__(EXPERT_THREADS)
expert_up_kernel(TA* __restrict__ mid, TA* __restrict__ smid, const TA* __restrict__ y, long long ldy, const TA* __restrict__ up,
                 const TA* __restrict__ sup, const int* __restrict__ idx, int T, int H, int ff, int sff, int top, int E, int act) {
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool is_shared = (int)blockIdx.x >= T * top;
    const int slot = is_shared ? (int)blockIdx.x - T * top : (int)blockIdx.x;
    const int t = is_shared ? slot : slot / top;
    const int rows = is_shared ? sff : ff;
    if ((int)blockIdx.y * EXPERT_ROWS >= rows) return;
    const bool vec = rows_vectorise(is_shared ? sup : up, H, H);
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < H; i += EXPERT_THREADS) smem[i] = to_float(y[(size_t)t * ldy + i]);
    const TA* base = sup;
    if (!is_shared) base = up + (size_t)min(max(idx[slot], 0), E - 1) * ff * H;
    __syncthreads();
    const int r = blockIdx.y * EXPERT_ROWS + warp;
    if (r < rows) {
        const float d = warp_sum(lane_dot<TA>(base + (size_t)r * H, smem, H, lane, vec));
        if (lane == 0) (is_shared ? smid : mid)[(size_t)slot * rows + r] = from_float<TA>(cellm_activate(d, act));
    }
}

// out[t, r] = sum_k wts[t, k] * (D_e mid[t * top + k])[r] (+ gate[t] * (D_s smid[t])[r]); down: [E * H, ff], D_s: [H, sff]
template <typename TA>
__global__ void __launch_bounds__(EXPERT_THREADS)
expert_down_kernel(TA* __restrict__ out, const TA* __restrict__ mid, const TA* __restrict__ smid, const TA* __restrict__ down,
                   const TA* __restrict__ sdown, const int* __restrict__ idx, const float* __restrict__ wts, const float* __restrict__ gate,
                   int H, int ff, int sff, int top, int E) {
    extern __shared__ __align__(16) float smem[];   // [top * ff] the token's middles, [sff] the shared expert's, then [top] weights and experts
    float* ms = smem;
    float* ss = smem + (size_t)top * ff;
    float* wk = ss + sff;
    int* ek = (int*)(wk + top);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const bool vec = rows_vectorise(down, ff, ff) && (ff & 3) == 0, svec = sdown && rows_vectorise(sdown, sff, sff) && ((top * ff) & 3) == 0;
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < top * ff; i += EXPERT_THREADS) ms[i] = to_float(mid[(size_t)t * top * ff + i]);
    if (sdown)
        for (int i = threadIdx.x; i < sff; i += EXPERT_THREADS) ss[i] = to_float(smid[(size_t)t * sff + i]);
    for (int k = threadIdx.x; k < top; k += EXPERT_THREADS) {
        wk[k] = wts[(size_t)t * top + k];
        ek[k] = min(max(idx[(size_t)t * top + k], 0), E - 1);
    }
    __syncthreads();
    const int r = blockIdx.y * EXPERT_ROWS + warp;
    if (r < H) {
        float a = 0.f;
#pragma unroll 2
        for (int k = 0; k < top; ++k) a += wk[k] * lane_dot<TA>(down + ((size_t)ek[k] * H + r) * ff, ms + (size_t)k * ff, ff, lane, vec);
        if (sdown) a += (gate ? gate[t] : 1.f) * lane_dot<TA>(sdown + (size_t)r * sff, ss, sff, lane, svec);
        a = warp_sum(a);
        if (lane == 0) out[(size_t)t * H + r] = from_float<TA>(a);
    }
}

// The chosen experts of every token, and the shared expert (sup null: none), walked row by row. mid: [T * top, ff] and
// smid: [T, sff], scratch of the activations' type. gate: [T] (null: the shared expert's result as it is).
CELLM_API int cellm_experts_rowwise(void* out, void* mid, void* smid, const void* y, long long ldy, const void* up, const void* down,
                                    const void* sup, const void* sdown, const int* idx, const float* wts, const float* gate, int T, int H,
                                    int ff, int sff, int top, int E, int act, int dtype, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (H < 1 || ff < 1 || top < 1 || E < 1 || sff < 0) return CELLM_ERR_SIZE;
    if ((sup == nullptr) != (sdown == nullptr) || (sup && (sff < 1 || !smid))) return CELLM_ERR_ARG;
    if (!sup) sff = 0;
    const size_t smem_up = (size_t)H * sizeof(float), smem_down = ((size_t)top * ff + sff + 2 * top) * sizeof(float);
    if (smem_up > 200 * 1024 || smem_down > 200 * 1024) return CELLM_ERR_SIZE;
    const int up_rows = ff > sff ? ff : sff;
    const dim3 grid_up((unsigned)(T * top + (sup ? T : 0)), (unsigned)((up_rows + EXPERT_ROWS - 1) / EXPERT_ROWS));
    const dim3 grid_down((unsigned)T, (unsigned)((H + EXPERT_ROWS - 1) / EXPERT_ROWS));
    if (grid_up.y > 65535 || grid_down.y > 65535) return CELLM_ERR_SIZE;
#define GO(TA)                                                                                                                    \
    do {                                                                                                                          \
        static bool configured = false;                                                                                           \
        if (!configured && (smem_up > 48 * 1024 || smem_down > 48 * 1024)) {                                                      \
            cudaError_t e = cudaFuncSetAttribute(expert_up_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);  \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(expert_down_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) return (int)e;                                                                                  \
            configured = true;                                                                                                    \
        }                                                                                                                         \
        CELLM_RUN(expert_up_kernel<TA>, grid_up, EXPERT_THREADS, smem_up, stream, (TA*)mid, (TA*)smid, (const TA*)y, ldy, (const TA*)up,  \
                  (const TA*)sup, idx, T, H, ff, sff, top, E, act);                                                               \
        CELLM_RUN(expert_down_kernel<TA>, grid_down, EXPERT_THREADS, smem_down, stream, (TA*)out, (const TA*)mid, (const TA*)smid, \
                  (const TA*)down, (const TA*)sdown, idx, wts, gate, H, ff, sff, top, E);                                         \
    } while (0)
    if (dtype == CELLM_F32) GO(float);
    else if (dtype == CELLM_BF16) GO(__nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef GO
    return CELLM_OK;
}

// ---- a plain activation: h = act(u) for 32-bit sums u [T, n] (row pitch ld) ----------------------------------------------
template <typename T>
__global__ void activation_kernel(T* __restrict__ h, const float* __restrict__ u, long long ld, int n, int act, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / n, c = i - t * n;
    h[i] = from_float<T>(cellm_activate(u[t * ld + c], act));
}

CELLM_API int cellm_activation(void* h, const float* u, long long ld, int T, int n, int act, int dtype, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return CELLM_OK;
    if (act < 0 || act > 3) return CELLM_ERR_ARG;
    const size_t total = (size_t)T * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == CELLM_F32) CELLM_RUN(activation_kernel<float>, blocks, 256, 0, stream, (float*)h, u, ld, n, act, total);
    else if (dtype == CELLM_BF16) CELLM_RUN(activation_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)h, u, ld, n, act, total);
    else return CELLM_ERR_DTYPE;
    return CELLM_OK;
}

// ---- many tokens: the (token, choice) slots sorted by expert ------------------------------------------------------------
// For the grouped tensor-core product every expert's slots form one run of rows, padded to whole tiles of 128 rows, in
// the order of the slots themselves (so a row's place depends on the step's tokens alone, never on timing).
#define MOE_TILE 128
#define MOE_SORT_THREADS 256

// One block an expert: it counts the slots of every expert (a histogram in shared memory), finds where its own run
// begins, names its tiles, and places its slots in their order. row_slot[row] = slot or -1 (padding); slot_row[slot] = row;
// tile_group[tile] = expert or -1 (behind the last run).
__global__ void __launch_bounds__(MOE_SORT_THREADS)
moe_sort_kernel(int* __restrict__ row_slot, int* __restrict__ slot_row, int* __restrict__ tile_group, const int* __restrict__ idx, int S,
                int E, int max_tiles) {
    extern __shared__ int sh[];
    int* hist = sh;             // [E]
    int* wsum = sh + E;         // [warps]
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = MOE_SORT_THREADS / 32;
    pdl_trigger();
    pdl_wait();
    for (int i = tid; i < E; i += MOE_SORT_THREADS) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < S; i += MOE_SORT_THREADS) {
        const int x = idx[i];
        if (x >= 0 && x < E) atomicAdd(&hist[x], 1);
    }
    __syncthreads();
    int start = 0;
    for (int f = 0; f < e; ++f) start += (hist[f] + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    const int count = hist[e], padded = (count + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    for (int i = tid; i < padded / MOE_TILE; i += MOE_SORT_THREADS) tile_group[start / MOE_TILE + i] = e;
    if (e == E - 1)
        for (int i = (start + padded) / MOE_TILE + tid; i < max_tiles; i += MOE_SORT_THREADS) tile_group[i] = -1;
    for (int i = count + tid; i < padded; i += MOE_SORT_THREADS) row_slot[start + i] = -1;
    int base = 0;
    for (int c0 = 0; c0 < S; c0 += MOE_SORT_THREADS) {
        const int i = c0 + tid;
        const bool mine = i < S && idx[i] == e;
        const unsigned b = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) wsum[warp] = __popc(b);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < nwarps; ++w) {
            if (w < warp) before += wsum[w];
            total += wsum[w];
        }
        if (mine) {
            const int r = start + base + before + __popc(b & ((1u << lane) - 1u));
            row_slot[r] = i;
            slot_row[i] = r;
        }
        base += total;
        __syncthreads();
    }
}

CELLM_API int cellm_moe_sort(int* row_slot, int* slot_row, int* tile_group, const int* idx, int S, int E, int max_tiles, cudaStream_t stream) {
    if (S <= 0) return CELLM_OK;
    if (E < 1 || max_tiles < 1 || E > 8192) return CELLM_ERR_SIZE;
    CELLM_RUN(moe_sort_kernel, E, MOE_SORT_THREADS, (size_t)(E + 32) * sizeof(int), stream, row_slot, slot_row, tile_group, idx, S, E, max_tiles);
    return CELLM_OK;
}

// xs[row, :] = y[row_slot[row] / top, :] for the rows of the named tiles (zeros in padding rows); 16-byte pieces.
__global__ void moe_gather_kernel(uint4* __restrict__ xs, const uint4* __restrict__ y, long long ldy16, const int* __restrict__ row_slot,
                                  const int* __restrict__ tile_group, int top, int H16) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    if (tile_group[row / MOE_TILE] < 0) return;
    const int slot = row_slot[row];
    uint4* dst = xs + (size_t)row * H16;
    if (slot < 0) {
        for (int i = threadIdx.x; i < H16; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* src = y + (size_t)(slot / top) * ldy16;
    for (int i = threadIdx.x; i < H16; i += blockDim.x) dst[i] = src[i];
}

// rows: the sorted buffer's rows (a multiple of 128); y: [T, H] bfloat16 with H a multiple of 8.
CELLM_API int cellm_moe_gather(void* xs, const void* y, long long ldy, const int* row_slot, const int* tile_group, int rows, int top, int H,
                               cudaStream_t stream) {
    if (rows <= 0) return CELLM_OK;
    if ((H & 7) || (ldy & 7) || (rows % MOE_TILE) || top < 1) return CELLM_ERR_SIZE;
    if (((uintptr_t)xs | (uintptr_t)y) & 15) return CELLM_ERR_ALIGN;
    CELLM_RUN(moe_gather_kernel, rows, 128, 0, stream, (uint4*)xs, (const uint4*)y, ldy / 8, row_slot, tile_group, top, H / 8);
    return CELLM_OK;
}

// out[t, :] = sum_k wts[t, k] * Y[slot_row[t * top + k], :] (+ gate[t] * shared[t, :]), the sum in the order of k, 32-bit.
__global__ void moe_combine_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ Y, const int* __restrict__ slot_row,
                                   const float* __restrict__ wts, const float* __restrict__ shared, const float* __restrict__ gate, int H,
                                   int top) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float g = shared ? (gate ? gate[t] : 1.f) : 0.f;
    for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
        float a0 = 0.f, a1 = 0.f;
        for (int k = 0; k < top; ++k) {
            const float w = wts[(size_t)t * top + k];
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Y + (size_t)slot_row[(size_t)t * top + k] * H + c));
            a0 += w * v.x;
            a1 += w * v.y;
        }
        if (shared) {
            a0 += g * shared[(size_t)t * H + c];
            a1 += g * shared[(size_t)t * H + c + 1];
        }
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * H + c) = __floats2bfloat162_rn(a0, a1);
    }
}

CELLM_API int cellm_moe_combine(void* out, const void* Y, const int* slot_row, const float* wts, const float* shared, const float* gate, int T,
                                int H, int top, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if ((H & 1) || top < 1) return CELLM_ERR_SIZE;
    CELLM_RUN(moe_combine_kernel, T, 256, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)Y, slot_row, wts, shared, gate, H, top);
    return CELLM_OK;
}
