// What stands between the q/k/v projection and an attention without a rotation: the RMS norm of the queries and
// of the keys - per head with one weight [d] for all heads, or over the whole projection with a weight of that
// size - an optional warm-up factor on the queries that grows with the logarithm of the position,
//     q *= 1 + coef * ln(floor((p + 1) / every) + 1),
// and the stores: queries to [T, QH, d], normalised keys and the values into the token's place in the paged cache.
// The values are a projection of their own, or the keys as projected (before their norm).  A layer that reads
// another layer's keys and values prepares its queries only.  One CTA per token; arithmetic in float.
#include "common.cuh"

#define HP_THREADS 128

// sum of squares of `n` floats in shared memory by the whole CTA (n == width of a group that spans all heads)
__device__ __forceinline__ float hp_block_sumsq(const float* v, int n, float* red) {
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += v[i] * v[i];
    return block_sum(ss, red);
}

// x [T, stride]: queries at column 0 (QH*d), keys behind them (KH*d), then the values (KH*dv) unless they are the keys.
// q_group / k_group: the width one norm spans (d: per head, weight [d]; QH*d or KH*d: the whole projection, weight of
// that size).  kv_slot null: nothing is stored and the keys are not read.
template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(HP_THREADS)
norm_heads_append_kernel(const TA* __restrict__ x, long long stride, const TW* __restrict__ qw, const TW* __restrict__ kw,
                         const int* __restrict__ positions, const int* __restrict__ kv_slot, TA* __restrict__ q_out,
                         TC* __restrict__ cache, int QH, int KH, int d, int dv, int q_group, int k_group, int values_are_keys,
                         int page_size, float eps, float temp_coef, int temp_every) {
    extern __shared__ float sm[];                              // q [QH*d] | k [KH*d]
    __shared__ float red[32];
    __shared__ float inv_q[64], inv_k[64];                     // per-head factors (per-head norms of up to 64 heads a pass)
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int nq = QH * d, nk = KH * d;
    const TA* xr = x + (size_t)t * stride;
    float* sq = sm;
    float* sk = sm + nq;
    const int slot = kv_slot ? kv_slot[t] : -1;
    const bool store = slot >= 0;                              // a padding row of a captured step stores nothing
    for (int i = threadIdx.x; i < nq; i += blockDim.x) sq[i] = to_f32(xr[i]);
    if (store) for (int i = threadIdx.x; i < nk; i += blockDim.x) sk[i] = to_f32(xr[nq + i]);
    __syncthreads();
    float temp = 1.0f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f);

    // ---- queries
    if (q_group == nq) {
        const float f = temp / sqrtf(hp_block_sumsq(sq, nq, red) / (float)nq + eps);
        for (int i = threadIdx.x; i < nq; i += blockDim.x)
            q_out[(size_t)t * nq + i] = from_f32<TA>(sq[i] * f * to_f32(qw[i]));
    } else {
        for (int h0 = 0; h0 < QH; h0 += 64) {
            for (int h = h0 + warp; h < min(QH, h0 + 64); h += nwarps) {
                float ss = 0.0f;
                for (int i = lane; i < d; i += 32) ss += sq[h * d + i] * sq[h * d + i];
                ss = warp_sum(ss);
                if (lane == 0) inv_q[h - h0] = temp / sqrtf(ss / (float)d + eps);
            }
            __syncthreads();
            const int n = min(QH - h0, 64) * d;
            for (int i = threadIdx.x; i < n; i += blockDim.x)
                q_out[(size_t)t * nq + h0 * d + i] = from_f32<TA>(sq[h0 * d + i] * inv_q[i / d] * to_f32(qw[i % d]));
            __syncthreads();
        }
    }
    if (!store) return;

    // ---- keys and values into the token's place: page [K: KH x page x d | V: KH x page x dv]
    const int page = slot / page_size, off = slot % page_size;
    const size_t page_stride = (size_t)KH * page_size * (d + dv);
    TC* kdst = cache + (size_t)page * page_stride + (size_t)off * d;
    TC* vdst = cache + (size_t)page * page_stride + (size_t)KH * page_size * d + (size_t)off * dv;
    if (values_are_keys) {
        for (int i = threadIdx.x; i < nk; i += blockDim.x)
            vdst[(size_t)(i / d) * page_size * dv + i % d] = from_f32<TC>(sk[i]);
    } else {
        const TA* xv = xr + nq + nk;
        for (int i = threadIdx.x; i < KH * dv; i += blockDim.x)
            vdst[(size_t)(i / dv) * page_size * dv + i % dv] = from_f32<TC>(to_f32(xv[i]));
    }
    if (k_group == nk) {
        const float f = 1.0f / sqrtf(hp_block_sumsq(sk, nk, red) / (float)nk + eps);
        for (int i = threadIdx.x; i < nk; i += blockDim.x)
            kdst[(size_t)(i / d) * page_size * d + i % d] = from_f32<TC>(sk[i] * f * to_f32(kw[i]));
    } else {
        for (int h0 = 0; h0 < KH; h0 += 64) {
            for (int h = h0 + warp; h < min(KH, h0 + 64); h += nwarps) {
                float ss = 0.0f;
                for (int i = lane; i < d; i += 32) ss += sk[h * d + i] * sk[h * d + i];
                ss = warp_sum(ss);
                if (lane == 0) inv_k[h - h0] = 1.0f / sqrtf(ss / (float)d + eps);
            }
            __syncthreads();
            const int n = min(KH - h0, 64) * d;
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const int h = h0 + i / d;
                kdst[(size_t)h * page_size * d + i % d] = from_f32<TC>(sk[h * d + i % d] * inv_k[i / d] * to_f32(kw[i % d]));
            }
            __syncthreads();
        }
    }
}

// The same for norms per head over heads of at most 256: a warp per (token, head), straight from global memory to
// the destinations, no shared memory and no block-wide barrier.  Units of a token: its query heads, its key heads, and
// (values of their own) its value heads.
#define HPW_WARPS 8
// V consecutive elements of a row as floats (V = 4: one 8-byte or 16-byte access; V = 1: one element)
template <int V> __device__ __forceinline__ void hp_load(const bf16* p, float (&v)[V]) {
    if (V == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
        v[0] = a.x; v[1] = a.y; v[V > 2 ? 2 : 0] = b.x; v[V > 3 ? 3 : 0] = b.y;
    } else {
        v[0] = __bfloat162float(p[0]);
    }
}
template <int V> __device__ __forceinline__ void hp_load(const float* p, float (&v)[V]) {
    if (V == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[V > 2 ? 2 : 0] = a.z; v[V > 3 ? 3 : 0] = a.w;
    } else {
        v[0] = p[0];
    }
}
template <int V> __device__ __forceinline__ void hp_store(bf16* p, const float (&v)[V]) {
    if (V == 4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[V > 2 ? 2 : 0], v[V > 3 ? 3 : 0]);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = pk;
    } else {
        p[0] = __float2bfloat16_rn(v[0]);
    }
}
template <int V> __device__ __forceinline__ void hp_store(float* p, const float (&v)[V]) {
    if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[V > 2 ? 2 : 0], v[V > 3 ? 3 : 0]);
    else p[0] = v[0];
}

// V: elements a lane takes at a time (4 where the head sizes are multiples of 4 and everything is aligned, else 1);
// M: passes of 32 * V elements that cover a head of at most 256.
template <typename TA, typename TW, int V, int M>
__global__ void __launch_bounds__(HPW_WARPS * 32)
norm_heads_append_warp_kernel(const TA* __restrict__ x, long long stride, const TW* __restrict__ qw, const TW* __restrict__ kw,
                              const int* __restrict__ positions, const int* __restrict__ kv_slot, TA* __restrict__ q_out,
                              TA* __restrict__ cache, int T, int QH, int KH, int d, int dv, int values_are_keys, int page_size,
                              float eps, float temp_coef, int temp_every) {
    pdl_trigger(); pdl_wait();
    const int lane = threadIdx.x & 31;
    const int per_tok = QH + (kv_slot ? KH + (values_are_keys ? 0 : KH) : 0);
    const size_t page_stride = (size_t)KH * page_size * (d + dv);
    const int t = blockIdx.x;                                  // a token per grid column, its heads over grid.y and the warps
    for (int idx = blockIdx.y * HPW_WARPS + (threadIdx.x >> 5); idx < per_tok; idx += gridDim.y * HPW_WARPS) {
        const TA* xr = x + (size_t)t * stride;
        const int slot = (idx >= QH) ? kv_slot[t] : 0;
        if (slot < 0) continue;                                // a padding row of a captured step stores nothing
        const int page = slot / page_size, off = slot % page_size;
        if (idx >= QH + KH) {                                  // a value head of its own: a copy
            const int hv = idx - QH - KH;
            const TA* src = xr + (size_t)(QH + KH) * d + (size_t)hv * dv;
            TA* vdst = cache + (size_t)page * page_stride + (size_t)KH * page_size * d + ((size_t)hv * page_size + off) * dv;
            for (int i = lane * V; i < dv; i += 32 * V) { float c[V]; hp_load<V>(src + i, c); hp_store<V>(vdst + i, c); }
            continue;
        }
        const bool is_q = idx < QH;
        const int hk = idx - QH;
        const TA* src = is_q ? xr + (size_t)idx * d : xr + (size_t)QH * d + (size_t)hk * d;
        float v[M][V];
        float ss = 0.0f;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int i = (lane + 32 * m) * V;
            if (i < d) hp_load<V>(src + i, v[m]);
            else {
#pragma unroll
                for (int c = 0; c < V; ++c) v[m][c] = 0.0f;
            }
#pragma unroll
            for (int c = 0; c < V; ++c) ss += v[m][c] * v[m][c];
        }
        ss = warp_sum(ss);
        float f = 1.0f / sqrtf(ss / (float)d + eps);
        if (is_q && temp_every > 0) f *= 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f);
        const TW* wn = is_q ? qw : kw;
        TA* dst = is_q ? q_out + ((size_t)t * QH + idx) * d
                       : cache + (size_t)page * page_stride + ((size_t)hk * page_size + off) * d;
        TA* vdst = cache + (size_t)page * page_stride + (size_t)KH * page_size * d + ((size_t)hk * page_size + off) * dv;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int i = (lane + 32 * m) * V;
            if (i < d) {
                float wv[V], o[V];
                hp_load<V>(wn + i, wv);
#pragma unroll
                for (int c = 0; c < V; ++c) o[c] = v[m][c] * f * wv[c];
                hp_store<V>(dst + i, o);
                if (!is_q && values_are_keys) hp_store<V>(vdst + i, v[m]);
            }
        }
    }
}

extern "C" int rb_norm_heads_append(const void* x, long long stride, int dtype, const void* qw, const void* kw, int w_dtype,
                                    const int* positions, const int* kv_slot, void* q_out, void* cache,
                                    int T, int QH, int KH, int d, int dv, int q_group, int k_group, int values_are_keys,
                                    int page_size, float eps, float temp_coef, int temp_every, void* stream) {
    if (T <= 0) return 0;
    if (QH <= 0 || KH <= 0 || d <= 0 || dv <= 0) RB_REFUSE("norm_heads_append: %d query heads, %d key heads of %d, values of %d", QH, KH, d, dv);
    if (q_group != d && q_group != QH * d) RB_REFUSE("norm_heads_append: a query norm over %d of %d x %d", q_group, QH, d);
    if (kv_slot && k_group != d && k_group != KH * d) RB_REFUSE("norm_heads_append: a key norm over %d of %d x %d", k_group, KH, d);
    if (values_are_keys && dv != d) RB_REFUSE("norm_heads_append: values that are the keys have the keys' size");
    if (temp_every > 0 && !positions) RB_REFUSE("norm_heads_append: the queries' warm-up needs the positions");
    if (kv_slot && (!cache || page_size <= 0 || !kw)) RB_REFUSE("norm_heads_append: storing needs a cache, a page size and the keys' norm");
    if (!qw) RB_REFUSE("norm_heads_append: the queries' norm weight is missing");
    cudaStream_t s = (cudaStream_t)stream;
    if (q_group == d && (!kv_slot || k_group == d) && d <= 256) {
        // norms per head: a warp per (token, head)
        const int per_tok = QH + (kv_slot ? KH * (values_are_keys ? 1 : 2) : 0);
        const dim3 blocks(T, (per_tok + HPW_WARPS - 1) / HPW_WARPS < 65535 ? (per_tok + HPW_WARPS - 1) / HPW_WARPS : 65535);
#define RB_HPW(TA, TW) do { \
            if (vec4) return rb_launch(norm_heads_append_warp_kernel<TA, TW, 4, 2>, blocks, dim3(HPW_WARPS * 32), 0, s, (const TA*)x, stride, \
                                       (const TW*)qw, (const TW*)kw, positions, kv_slot, (TA*)q_out, (TA*)cache, T, QH, KH, d, dv, \
                                       values_are_keys, page_size, eps, temp_coef, temp_every); \
            return rb_launch(norm_heads_append_warp_kernel<TA, TW, 1, 8>, blocks, dim3(HPW_WARPS * 32), 0, s, (const TA*)x, stride, \
                             (const TW*)qw, (const TW*)kw, positions, kv_slot, (TA*)q_out, (TA*)cache, T, QH, KH, d, dv, \
                             values_are_keys, page_size, eps, temp_coef, temp_every); } while (0)
        const bool vec4 = d % 4 == 0 && dv % 4 == 0 && stride % 4 == 0 &&
            (((uintptr_t)x | (uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)qw | (uintptr_t)kw) & 15) == 0;
        if (dtype == RB_F32 && w_dtype == RB_F32) RB_HPW(float, float);
        if (dtype == RB_BF16 && w_dtype == RB_BF16) RB_HPW(bf16, bf16);
        if (dtype == RB_BF16 && w_dtype == RB_F32) RB_HPW(bf16, float);
#undef RB_HPW
        RB_REFUSE("norm_heads_append: dtypes %d, %d", dtype, w_dtype);
    }
    const size_t smem = (size_t)(QH + KH) * d * sizeof(float);
    if (smem > 200 * 1024) RB_REFUSE("norm_heads_append: %d floats of queries and keys per token", (QH + KH) * d);
#define RB_HP(TA, TW) do { \
        if (smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(norm_heads_append_kernel<TA, TW, TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
        } \
        return rb_launch(norm_heads_append_kernel<TA, TW, TA>, dim3(T), dim3(HP_THREADS), smem, s, (const TA*)x, stride, \
                         (const TW*)qw, (const TW*)kw, positions, kv_slot, (TA*)q_out, (TA*)cache, QH, KH, d, dv, q_group, k_group, \
                         values_are_keys, page_size, eps, temp_coef, temp_every); } while (0)
    if (dtype == RB_F32 && w_dtype == RB_F32) RB_HP(float, float);
    if (dtype == RB_BF16 && w_dtype == RB_BF16) RB_HP(bf16, bf16);
    if (dtype == RB_BF16 && w_dtype == RB_F32) RB_HP(bf16, float);
#undef RB_HP
    RB_REFUSE("norm_heads_append: dtypes %d, %d", dtype, w_dtype);
}
