// Short causal convolution over time, each channel alone, for batches of request portions:
//   y[t, c] = act( sum_j w[c, j] * u[t - taps + 1 + j, c] ),   j = 0 .. taps-1 (the last tap is the present token)
// Inputs before a request's first token are zero; inputs before the portion's first token come from the
// request's slot, which holds its last taps-1 inputs, oldest first: state [slots, taps-1, C] float.
// A thread owns one channel of one request over a segment of RC_SEG tokens and slides a register window
// along it, so a token's result is the same chain of FMAs (ascending j) however the request was cut.
// Where every request of the step fits one segment the same thread also leaves the new window in the
// slot; else a second small kernel does, after all reads of the old one.
#include "common.cuh"

#define RC_MAX_TAPS 8
#define RC_SEG 64
#define RC_THREADS 128

template <typename TA>
__global__ void __launch_bounds__(RC_THREADS)
shortconv_kernel(const TA* __restrict__ u, long long ldu, const float* __restrict__ w, float* __restrict__ state,
                 TA* __restrict__ y, long long ldy, const int* __restrict__ cu_q, const int* __restrict__ entry_slot,
                 int C, int taps, int act, int update) {
    pdl_trigger();
    const int c = blockIdx.x * RC_THREADS + threadIdx.x;
    // taps and window sit at the END of fixed arrays (the present token's tap last); the places in front hold zeros
    const int lead = RC_MAX_TAPS - taps;
    float wv[RC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS; ++j) wv[j] = (c < C && j >= lead) ? w[(size_t)c * taps + (j - lead)] : 0.0f;
    pdl_wait();
    if (c >= C) return;
    const int e = blockIdx.y;
    const int s0 = cu_q[e], n = cu_q[e + 1] - s0;
    const int a = blockIdx.z * RC_SEG;
    if (a >= n) return;
    const int hist = taps - 1;
    float* st = state + (size_t)entry_slot[e] * hist * C + c;
    float win[RC_MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS - 1; ++j) {
        win[j] = 0.0f;
        if (j >= lead) {
            const int idx = a - (RC_MAX_TAPS - 1) + j;    // local index of the input this window place holds (< a)
            win[j] = idx < 0 ? st[(size_t)(hist + idx) * C] : to_f32(u[(size_t)(s0 + idx) * ldu + c]);
        }
    }
    const int end = min(a + RC_SEG, n);
    for (int i = a; i < end; ++i) {
        const float cur = to_f32(u[(size_t)(s0 + i) * ldu + c]);
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS - 1; ++j) acc = fmaf(wv[j], win[j], acc);
        acc = fmaf(wv[RC_MAX_TAPS - 1], cur, acc);
        if (act == 1) acc = acc / (1.0f + expf(-acc));
        y[(size_t)(s0 + i) * ldy + c] = from_f32<TA>(acc);
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS - 2; ++j) win[j] = win[j + 1];
        win[RC_MAX_TAPS - 2] = cur;
    }
    if (update) {
#pragma unroll
        for (int j = 0; j < RC_MAX_TAPS - 1; ++j) if (j >= lead) st[(size_t)(j - lead) * C] = win[j];
    }
}

// The slot's window after a step whose requests span several segments: the last taps-1 inputs of (old window, u).
template <typename TA>
__global__ void __launch_bounds__(RC_THREADS)
shortconv_state_kernel(const TA* __restrict__ u, long long ldu, float* __restrict__ state, const int* __restrict__ cu_q,
                       const int* __restrict__ entry_slot, int C, int taps) {
    pdl_trigger(); pdl_wait();
    const int c = blockIdx.x * RC_THREADS + threadIdx.x;
    if (c >= C) return;
    const int e = blockIdx.y;
    const int s0 = cu_q[e], n = cu_q[e + 1] - s0;
    const int hist = taps - 1;
    float* st = state + (size_t)entry_slot[e] * hist * C + c;
    float win[RC_MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS - 1; ++j) {
        win[j] = 0.0f;
        if (j < hist) {
            const int idx = n - hist + j;
            win[j] = idx < 0 ? st[(size_t)(hist + idx) * C] : to_f32(u[(size_t)(s0 + idx) * ldu + c]);
        }
    }
#pragma unroll
    for (int j = 0; j < RC_MAX_TAPS - 1; ++j) if (j < hist) st[(size_t)j * C] = win[j];
}

// u [T, C] (row stride ldu), y [T, C] (row stride ldy), w [C, taps] float, state [slots, taps-1, C] float,
// cu_q [E+1], entry_slot [E]; max_q_len: the longest portion of the step.  act 0: none, 1: silu.
extern "C" int rb_shortconv(const void* u, long long ldu, const float* w, float* state, void* y, long long ldy, int dtype,
                            const int* cu_q, const int* entry_slot, int n_entries, int max_q_len, int C, int taps, int act,
                            void* stream) {
    if (n_entries <= 0 || max_q_len <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > RC_MAX_TAPS) RB_REFUSE("shortconv: %d channels, %d taps (1..%d)", C, taps, RC_MAX_TAPS);
    if (act != 0 && act != 1) RB_REFUSE("shortconv: activation %d", act);
    cudaStream_t s = (cudaStream_t)stream;
    const int nseg = rb_ceil_div(max_q_len, RC_SEG);
    const int update = nseg == 1 ? 1 : 0;
    dim3 grid(rb_ceil_div(C, RC_THREADS), n_entries, nseg);
    int rc;
    if (dtype == RB_F32) rc = rb_launch(shortconv_kernel<float>, grid, dim3(RC_THREADS), 0, s, (const float*)u, ldu, w, state, (float*)y, ldy, cu_q, entry_slot, C, taps, act, update);
    else if (dtype == RB_BF16) rc = rb_launch(shortconv_kernel<bf16>, grid, dim3(RC_THREADS), 0, s, (const bf16*)u, ldu, w, state, (bf16*)y, ldy, cu_q, entry_slot, C, taps, act, update);
    else RB_REFUSE("shortconv: dtype %d", dtype);
    if (rc || update || taps == 1) return rc;
    dim3 g2(rb_ceil_div(C, RC_THREADS), n_entries);
    if (dtype == RB_F32) return rb_launch(shortconv_state_kernel<float>, g2, dim3(RC_THREADS), 0, s, (const float*)u, ldu, state, cu_q, entry_slot, C, taps);
    return rb_launch(shortconv_state_kernel<bf16>, g2, dim3(RC_THREADS), 0, s, (const bf16*)u, ldu, state, cu_q, entry_slot, C, taps);
}

// ------------------------------------------------------------------ heads to unit root mean square, and into the cache
// x [T, (QH + KH) * dk + KH * dv] (row stride ldx): q heads, k heads, v heads of a token.
//   q -> q / sqrt(mean(q^2) + eps) -> q_out [T, QH, dk]          (no weight)
//   k -> the same                   -> the K part of the token's cache slot
//   v -> copy                       -> the V part
// Cache of one layer: [page][ K: [KH][page_size][dk] | V: [KH][page_size][dv] ]; slot = page * page_size + offset,
// slot < 0: nothing is stored.  One warp per (token, head).
template <typename TA, typename TC>
__global__ void unit_heads_append_kernel(const TA* __restrict__ x, long long ldx, const int* __restrict__ kv_slot,
                                         TA* __restrict__ q_out, TC* __restrict__ cache, int n_tokens, int QH, int KH,
                                         int dk, int dv, int page_size, float eps) {
    pdl_trigger(); pdl_wait();
    const int heads = QH + 2 * KH;
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wg >= (long long)n_tokens * heads) return;
    const int t = (int)(wg / heads), hh = (int)(wg % heads);
    const int slot = kv_slot ? kv_slot[t] : -1;
    const size_t page_elems = (size_t)KH * page_size * (dk + dv);
    if (hh >= QH + KH) {
        if (slot < 0) return;
        const int kh = hh - QH - KH;
        const TA* src = x + (size_t)t * ldx + (size_t)(QH + KH) * dk + (size_t)kh * dv;
        TC* dst = cache + (size_t)(slot / page_size) * page_elems + (size_t)KH * page_size * dk +
                  ((size_t)kh * page_size + slot % page_size) * dv;
        for (int i = lane; i < dv; i += 32) dst[i] = from_f32<TC>(to_f32(src[i]));
        return;
    }
    const bool is_q = hh < QH;
    if (!is_q && slot < 0) return;
    const TA* src = x + (size_t)t * ldx + (size_t)hh * dk;
    float ss = 0.0f;
    for (int i = lane; i < dk; i += 32) { const float v = to_f32(src[i]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)dk + eps);
    if (is_q) {
        TA* dst = q_out + ((size_t)t * QH + hh) * dk;
        for (int i = lane; i < dk; i += 32) dst[i] = from_f32<TA>(to_f32(src[i]) * rstd);
    } else {
        const int kh = hh - QH;
        TC* dst = cache + (size_t)(slot / page_size) * page_elems + ((size_t)kh * page_size + slot % page_size) * dk;
        for (int i = lane; i < dk; i += 32) dst[i] = from_f32<TC>(to_f32(src[i]) * rstd);
    }
}
extern "C" int rb_unit_heads_append(const void* x, long long ldx, const int* kv_slot, void* q_out, void* cache, int dtype,
                                    int n_tokens, int QH, int KH, int dk, int dv, int page_size, float eps, void* stream) {
    if (n_tokens <= 0) return 0;
    if (QH <= 0 || KH <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) RB_REFUSE("unit_heads_append: heads %d/%d sizes %d/%d page %d", QH, KH, dk, dv, page_size);
    const int blocks = rb_ceil_div((long long)n_tokens * (QH + 2 * KH), 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RB_F32) return rb_launch(unit_heads_append_kernel<float, float>, dim3(blocks), dim3(128), 0, s, (const float*)x, ldx, kv_slot, (float*)q_out, (float*)cache, n_tokens, QH, KH, dk, dv, page_size, eps);
    if (dtype == RB_BF16) return rb_launch(unit_heads_append_kernel<bf16, bf16>, dim3(blocks), dim3(128), 0, s, (const bf16*)x, ldx, kv_slot, (bf16*)q_out, (bf16*)cache, n_tokens, QH, KH, dk, dv, page_size, eps);
    RB_REFUSE("unit_heads_append: dtype %d", dtype);
}
