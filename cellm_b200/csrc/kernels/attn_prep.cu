// Queries, keys and values on their way from the projection into the attention, in the general form: an RMS
// norm of queries and keys taken per head or over the whole projection (all heads of a token at once), a
// query temperature that grows with the position, keys and values of different widths, and the write of keys
// and values into the request's pages. (The per-head norm with a rotation is qk_norm_rope.cu's.)
//
//   span 0: no norm;  span 1: every head by its own root mean square (weights [hd], the same for every head);
//   span 2: all heads of a token by one root mean square (weights [heads * hd])
//   q <- q * (1 + coef * ln(floor((pos + 1) / every) + 1))     (coef = 0: no temperature)
//
// Norm, temperature and positions are 32-bit. Rows of the projection: [nh * hd | nkv * hd | nkv * hdv].
// Cache layout of one layer: keys [page][kv_head][slot in page][hq], values [page][kv_head][slot in page][hv], where
// hq >= hd and hv >= hdv are the widths the rows are kept in: a head padded with zeros to a width the fast attention
// kernels take gives the same scores (the zeros add nothing) and values whose last columns are zero.
#include "common.cuh"

#define PREP_THREADS 256

template <typename TA, typename TW>
__global__ void __launch_bounds__(PREP_THREADS)
attn_prep_kernel(TA* __restrict__ q_out, const TA* __restrict__ qkv, long long row_stride, const TW* __restrict__ q_w,
                 const TW* __restrict__ k_w, float eps, int span, float temp_coef, int temp_every,
                 const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                 int bt_stride, TA* __restrict__ k_pool, TA* __restrict__ v_pool, int num_pages, int page_size, int nh, int nkv,
                 int hd, int hdv, int hq, int hv, int* __restrict__ err) {
    extern __shared__ float smem[];          // [nh + nkv] a head's sum of squares, then its factor
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = PREP_THREADS / 32;
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    float temp = 1.f;
    if (temp_coef != 0.f) temp = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
    long long page = -1;
    if (nkv > 0) {
        const int b = seq_of_token[t];
        const int p = block_table[(size_t)b * bt_stride + pos / page_size];
        if (p < 0 || p >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
        } else {
            page = p;
        }
    }
    pdl_wait();
    const TA* row = qkv + (size_t)t * row_stride;
    const int heads = nh + nkv;
    if (span != 0) {
        for (int h = warp; h < heads; h += nwarps) {
            const TA* src = row + (size_t)h * hd;
            float ss = 0.f;
            for (int i = lane; i < hd; i += 32) {
                const float v = to_float(src[i]);
                ss += v * v;
            }
            ss = warp_sum(ss);
            if (lane == 0) smem[h] = ss;
        }
        __syncthreads();
        float fq = 0.f, fk = 0.f;
        if (span == 2) {                     // every thread adds the heads' sums in the same order
            for (int h = 0; h < nh; ++h) fq += smem[h];
            for (int h = nh; h < heads; ++h) fk += smem[h];
            fq = 1.0f / sqrtf(fq / (float)(nh * hd) + eps);
            fk = nkv > 0 ? 1.0f / sqrtf(fk / (float)(nkv * hd) + eps) : 0.f;
        }
        __syncthreads();
        for (int h = threadIdx.x; h < heads; h += PREP_THREADS)
            smem[h] = span == 2 ? (h < nh ? fq : fk) : 1.0f / sqrtf(smem[h] / (float)hd + eps);
        __syncthreads();
    }
    // queries
    for (int o = threadIdx.x; o < nh * hq; o += PREP_THREADS) {
        const int h = o / hq, c = o - h * hq;
        float v = 0.f;
        if (c < hd) {
            const int i = h * hd + c;
            v = to_float(row[i]);
            if (span != 0) v = v * smem[h] * to_float(q_w[span == 2 ? i : c]);
            v *= temp;
        }
        q_out[(size_t)t * nh * hq + o] = from_float<TA>(v);
    }
    if (page < 0) return;
    const int slot = pos % page_size;
    // keys
    const TA* krow = row + (size_t)nh * hd;
    for (int o = threadIdx.x; o < nkv * hq; o += PREP_THREADS) {
        const int h = o / hq, c = o - h * hq;
        float v = 0.f;
        if (c < hd) {
            const int i = h * hd + c;
            v = to_float(krow[i]);
            if (span != 0) v = v * smem[nh + h] * to_float(k_w[span == 2 ? i : c]);
        }
        k_pool[((size_t)page * nkv + h) * page_size * hq + (size_t)slot * hq + c] = from_float<TA>(v);
    }
    // values
    const TA* vrow = krow + (size_t)nkv * hd;
    for (int o = threadIdx.x; o < nkv * hv; o += PREP_THREADS) {
        const int h = o / hv, c = o - h * hv;
        v_pool[((size_t)page * nkv + h) * page_size * hv + (size_t)slot * hv + c] = c < hdv ? vrow[h * hdv + c] : from_float<TA>(0.f);
    }
}

// The same in 16-byte pieces, for widths and pitches that are multiples of a piece (8 bfloat16 or 4 float values) and
// aligned rows. A thread's piece of q or k leaves its sum of squares in shared memory; one thread a head adds a head's
// pieces in their order, so the sums do not depend on how the threads ran.
template <typename TA, typename TW>
__global__ void __launch_bounds__(PREP_THREADS)
attn_prep_vec_kernel(TA* __restrict__ q_out, const TA* __restrict__ qkv, long long row_stride, const TW* __restrict__ q_w,
                     const TW* __restrict__ k_w, float eps, int span, float temp_coef, int temp_every,
                     const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                     int bt_stride, TA* __restrict__ k_pool, TA* __restrict__ v_pool, int num_pages, int page_size, int nh, int nkv,
                     int hd, int hdv, int hq, int hv, int* __restrict__ err) {
    constexpr int PER = 16 / (int)sizeof(TA);
    extern __shared__ float smem[];          // [nh + nkv] a head's factor, then [(nh + nkv) * hd / PER] the pieces' sums of squares
    const int heads = nh + nkv;
    float* part = smem + heads;
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    float temp = 1.f;
    if (temp_coef != 0.f) temp = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
    long long page = -1;
    if (nkv > 0) {
        const int b = seq_of_token[t];
        const int p = block_table[(size_t)b * bt_stride + pos / page_size];
        if (p < 0 || p >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, CELLM_DEV_BAD_PAGE);
        } else {
            page = p;
        }
    }
    pdl_wait();
    const TA* row = qkv + (size_t)t * row_stride;
    const int per_head = hd / PER;
    if (span != 0) {
        for (int c = threadIdx.x; c < heads * per_head; c += PREP_THREADS) {
            const uint4 x = *reinterpret_cast<const uint4*>(row + (size_t)c * PER);
            const TA* xp = reinterpret_cast<const TA*>(&x);
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < PER; ++k) { const float v = to_float(xp[k]); ss += v * v; }
            part[c] = ss;
        }
        __syncthreads();
        for (int h = threadIdx.x; h < heads; h += PREP_THREADS) {
            float ss = 0.f;
            for (int c = 0; c < per_head; ++c) ss += part[h * per_head + c];
            smem[h] = ss;
        }
        __syncthreads();
        float fq = 0.f, fk = 0.f;
        if (span == 2) {
            for (int h = 0; h < nh; ++h) fq += smem[h];
            for (int h = nh; h < heads; ++h) fk += smem[h];
            fq = 1.0f / sqrtf(fq / (float)(nh * hd) + eps);
            fk = nkv > 0 ? 1.0f / sqrtf(fk / (float)(nkv * hd) + eps) : 0.f;
        }
        __syncthreads();
        for (int h = threadIdx.x; h < heads; h += PREP_THREADS)
            smem[h] = span == 2 ? (h < nh ? fq : fk) : 1.0f / sqrtf(smem[h] / (float)hd + eps);
        __syncthreads();
    }
    // queries and keys: piece o of the kept rows (heads of hq values) from piece c of the projection (heads of hd)
    const int kept = hq / PER, slot = pos % page_size;
    const int n_out = (nh + (page >= 0 ? nkv : 0)) * kept;
    for (int o = threadIdx.x; o < n_out; o += PREP_THREADS) {
        const int h = o / kept, c = (o - h * kept) * PER;          // h: head among queries then keys
        __align__(16) TA y[PER];
#pragma unroll
        for (int k = 0; k < PER; ++k) y[k] = from_float<TA>(0.f);
        if (c < hd) {
            const uint4 x = *reinterpret_cast<const uint4*>(row + (size_t)h * hd + c);
            const TA* xp = reinterpret_cast<const TA*>(&x);
            const bool is_q = h < nh;
            const TW* w = is_q ? q_w : k_w;
            const int wi = span == 2 ? (is_q ? h : h - nh) * hd + c : c;
            const float f = (span != 0 ? smem[h] : 1.f);
#pragma unroll
            for (int k = 0; k < PER; ++k) {
                float v = to_float(xp[k]);
                if (span != 0) v = v * f * to_float(w[wi + k]);
                y[k] = from_float<TA>(is_q ? v * temp : v);
            }
        }
        TA* dst = h < nh ? q_out + (size_t)t * nh * hq + (size_t)h * hq + c
                         : k_pool + ((size_t)page * nkv + (h - nh)) * page_size * hq + (size_t)slot * hq + c;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(y);
    }
    if (page < 0) return;
    const TA* vrow = row + (size_t)heads * hd;
    const int vkept = hv / PER;
    for (int o = threadIdx.x; o < nkv * vkept; o += PREP_THREADS) {
        const int h = o / vkept, c = (o - h * vkept) * PER;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (c < hdv) x = *reinterpret_cast<const uint4*>(vrow + (size_t)h * hdv + c);
        *reinterpret_cast<uint4*>(v_pool + ((size_t)page * nkv + h) * page_size * hv + (size_t)slot * hv + c) = x;
    }
}

// qkv: [T, nh*hd + nkv*(hd + hdv)] (row pitch row_stride); q_out: [T, nh*hq]. nkv = 0: the rows hold queries only and
// nothing is written. Weights: [hd] (span 1) or [nh*hd] and [nkv*hd] (span 2), null with span 0. hq, hv: the widths
// queries and keys, and values, are kept in (0: as they are).
CELLM_API int cellm_attn_prep(void* q_out, const void* qkv, long long row_stride, const void* q_w, const void* k_w, int w_dtype, float eps,
                              int span, float temp_coef, int temp_every, const int* positions, const int* seq_of_token,
                              const int* block_table, int bt_stride, void* k_pool, void* v_pool, int num_pages, int page_size, int T,
                              int nh, int nkv, int hd, int hdv, int hq, int hv, int dtype, int* err, cudaStream_t stream) {
    if (T <= 0) return CELLM_OK;
    if (hq == 0) hq = hd;
    if (hv == 0) hv = hdv;
    if (hq < hd || hv < hdv) return CELLM_ERR_SIZE;
    if (nh < 1 || nkv < 0 || hd < 1 || hdv < 1 || span < 0 || span > 2) return CELLM_ERR_SIZE;
    if (span != 0 && (!q_w || (nkv > 0 && !k_w))) return CELLM_ERR_ARG;
    if (temp_coef != 0.f && temp_every < 1) return CELLM_ERR_ARG;
    if (nkv > 0 && (!block_table || !k_pool || !v_pool || page_size < 1)) return CELLM_ERR_ARG;
    const size_t smem = (size_t)(nh + nkv) * sizeof(float);
    {   // 16-byte pieces where every width and pitch is a multiple of a piece and the rows are aligned
        const int per = dtype == CELLM_F32 ? 4 : 8;
        const size_t vsmem = smem + (size_t)(nh + nkv) * (hd / per) * sizeof(float);
        const bool vec = (dtype == CELLM_F32 || dtype == CELLM_BF16) && hd % per == 0 && hdv % per == 0 && hq % per == 0 && hv % per == 0 &&
                         row_stride % per == 0 && vsmem <= 48 * 1024 &&
                         (((uintptr_t)q_out | (uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0;
        if (vec) {
#define GOV(TA, TW)                                                                                                          \
    CELLM_RUN((attn_prep_vec_kernel<TA, TW>), T, PREP_THREADS, vsmem, stream, (TA*)q_out, (const TA*)qkv, row_stride, (const TW*)q_w, \
              (const TW*)k_w, eps, span, temp_coef, temp_every, positions, seq_of_token, block_table, bt_stride, (TA*)k_pool,  \
              (TA*)v_pool, num_pages, page_size, nh, nkv, hd, hdv, hq, hv, err)
            if (dtype == CELLM_F32 && (w_dtype == CELLM_F32 || span == 0)) GOV(float, float);
            else if (dtype == CELLM_F32 && w_dtype == CELLM_BF16) GOV(float, __nv_bfloat16);
            else if (dtype == CELLM_BF16 && w_dtype == CELLM_F32) GOV(__nv_bfloat16, float);
            else if (dtype == CELLM_BF16 && (w_dtype == CELLM_BF16 || span == 0)) GOV(__nv_bfloat16, __nv_bfloat16);
            else return CELLM_ERR_DTYPE;
#undef GOV
            return CELLM_OK;
        }
    }
#define GO(TA, TW)                                                                                                           \
    CELLM_RUN((attn_prep_kernel<TA, TW>), T, PREP_THREADS, smem, stream, (TA*)q_out, (const TA*)qkv, row_stride, (const TW*)q_w, \
              (const TW*)k_w, eps, span, temp_coef, temp_every, positions, seq_of_token, block_table, bt_stride, (TA*)k_pool,  \
              (TA*)v_pool, num_pages, page_size, nh, nkv, hd, hdv, hq, hv, err)
    if (dtype == CELLM_F32 && (w_dtype == CELLM_F32 || span == 0)) GO(float, float);
    else if (dtype == CELLM_F32 && w_dtype == CELLM_BF16) GO(float, __nv_bfloat16);
    else if (dtype == CELLM_BF16 && w_dtype == CELLM_F32) GO(__nv_bfloat16, float);
    else if (dtype == CELLM_BF16 && (w_dtype == CELLM_BF16 || span == 0)) GO(__nv_bfloat16, __nv_bfloat16);
    else return CELLM_ERR_DTYPE;
#undef GO
    return CELLM_OK;
}
