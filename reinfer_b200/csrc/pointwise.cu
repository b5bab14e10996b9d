// Pointwise kernels that the statistics-free layers need: the Dynamic Tanh norm (with the
// residual sum in front, like the RMS norm of elementwise.cu), the soft cap on logits, a unary
// function on a strided block, and the per-head output stage of the recurrent mixers (unit root
// mean square over a head, weight, gate).  All arithmetic is 32-bit.
#include "common.cuh"

// ------------------------------------------------------------------ Dynamic Tanh
// x[r,:] += sum_s delta[s][r,:] (ascending s; x is float and is written back), then
// out[r,:] = tanh(alpha * x) * w + b.  No mean, no variance: nothing crosses a row.
// With row_idx the input row of output row r is row_idx[r] and x stays as it is.
template <typename TW, typename TO>
__global__ void dyt_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
                           const TW* __restrict__ w, const TW* __restrict__ b, const TW* __restrict__ alpha,
                           TO* __restrict__ out, const int* __restrict__ row_idx, int h) {
    pdl_trigger();
    const float a = to_f32(alpha[0]);                   // weights never change: read before the wait
    pdl_wait();
    const int r = blockIdx.x;
    const size_t in_row = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* xr = x + in_row * h;
    const bool keep = delta && !row_idx;
    TO* o = out + (size_t)r * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float v = xr[i];
        if (delta) {
            for (int s = 0; s < n_delta; ++s) v += delta[(size_t)s * delta_stride + in_row * h + i];
            if (keep) xr[i] = v;
        }
        o[i] = from_f32<TO>(fmaf(tanhf(a * v), to_f32(w[i]), to_f32(b[i])));
    }
}

extern "C" int rb_dyt(float* x, const float* delta, int n_delta, long long delta_stride, const void* w, const void* b,
                      const void* alpha, int w_dtype, void* out, int out_dtype, const int* row_idx, int rows, int h,
                      void* stream) {
    if (rows <= 0) return 0;
    if (h <= 0) RB_REFUSE("dyt: width %d", h);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = h >= 2048 ? 512 : (h >= 512 ? 256 : 128);
#define RB_DYT(TW, TO) return rb_launch(dyt_kernel<TW, TO>, dim3(rows), dim3(threads), 0, s, x, delta, n_delta, delta_stride, \
                                        (const TW*)w, (const TW*)b, (const TW*)alpha, (TO*)out, row_idx, h)
    if (w_dtype == RB_F32 && out_dtype == RB_F32) RB_DYT(float, float);
    if (w_dtype == RB_BF16 && out_dtype == RB_BF16) RB_DYT(bf16, bf16);
    if (w_dtype == RB_F32 && out_dtype == RB_BF16) RB_DYT(float, bf16);
    if (w_dtype == RB_BF16 && out_dtype == RB_F32) RB_DYT(bf16, float);
#undef RB_DYT
    RB_REFUSE("dyt: dtypes %d, %d", w_dtype, out_dtype);
}

// ------------------------------------------------------------------ soft cap
// x <- cap * tanh(x / cap), in place on float rows.
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_trigger(); pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}
extern "C" int rb_softcap(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.0f)) RB_REFUSE("softcap: cap %f", cap);
    return rb_launch(softcap_kernel, dim3(rb_ceil_div(n, 256)), dim3(256), 0, (cudaStream_t)stream, x, (size_t)n, cap);
}

// ------------------------------------------------------------------ unary function on a strided block
// x[r, c] <- f(x[r, c]) for r < rows, c < cols, row stride ld.  kind 0: tanh.
template <typename TA>
__global__ void unary_kernel(TA* __restrict__ x, long long ld, int rows, int cols, int kind) {
    pdl_trigger(); pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols) return;
    TA* p = x + (i / cols) * ld + (i % cols);
    const float v = to_f32(*p);
    *p = from_f32<TA>(kind == 0 ? tanhf(v) : v);
}
extern "C" int rb_unary(void* x, int dtype, long long ld, int rows, int cols, int kind, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (kind != 0) RB_REFUSE("unary: kind %d", kind);
    const int blocks = rb_ceil_div((long long)rows * cols, 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RB_F32) return rb_launch(unary_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)x, ld, rows, cols, kind);
    if (dtype == RB_BF16) return rb_launch(unary_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (bf16*)x, ld, rows, cols, kind);
    RB_REFUSE("unary: dtype %d", dtype);
}

// ------------------------------------------------------------------ per-head output stage
// o [T, H, dv] float (what a recurrence read out).  For every (token, head):
//   y = o / sqrt(mean(o^2) + eps) * w * act(gate) * out_scale
// w: [dv] shared by the heads (w_heads = 0) or [H * dv] (w_heads = 1).  gate [T, H * dv] with row stride ldg;
// act 0: sigmoid, 1: silu.  One warp per (token, head); a lane sums its strided elements in ascending order.
template <typename TA>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_heads,
                                      const TA* __restrict__ gate, long long ldg, int act, TA* __restrict__ out, long long ldo,
                                      int n_tokens, int H, int dv, float eps, float out_scale) {
    pdl_trigger(); pdl_wait();
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wg >= (long long)n_tokens * H) return;
    const int t = (int)(wg / H), hh = (int)(wg % H);
    const float* src = o + ((size_t)t * H + hh) * dv;
    float ss = 0.0f;
    for (int i = lane; i < dv; i += 32) { const float v = src[i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)dv + eps);
    const TA* g = gate + (size_t)t * ldg + (size_t)hh * dv;
    TA* dst = out + (size_t)t * ldo + (size_t)hh * dv;
    const float* wv = w + (w_heads ? (size_t)hh * dv : 0);
    for (int i = lane; i < dv; i += 32) {
        const float z = to_f32(g[i]);
        const float sg = 1.0f / (1.0f + expf(-z));
        const float gv = act == 1 ? z * sg : sg;
        dst[i] = from_f32<TA>(src[i] * rstd * wv[i] * gv * out_scale);
    }
}
extern "C" int rb_head_norm_gate(const float* o, const float* w, int w_heads, const void* gate, long long ldg, int act,
                                 void* out, long long ldo, int dtype, int n_tokens, int H, int dv, float eps, float out_scale,
                                 void* stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || dv <= 0) RB_REFUSE("head_norm_gate: %d heads of %d", H, dv);
    if (act != 0 && act != 1) RB_REFUSE("head_norm_gate: gate function %d", act);
    const int blocks = rb_ceil_div((long long)n_tokens * H, 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RB_F32) return rb_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, s, o, w, w_heads, (const float*)gate, ldg, act, (float*)out, ldo, n_tokens, H, dv, eps, out_scale);
    if (dtype == RB_BF16) return rb_launch(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(128), 0, s, o, w, w_heads, (const bf16*)gate, ldg, act, (bf16*)out, ldo, n_tokens, H, dv, eps, out_scale);
    RB_REFUSE("head_norm_gate: dtype %d", dtype);
}
