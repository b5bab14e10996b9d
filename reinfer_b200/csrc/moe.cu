// A mixture of small feed-forward experts, the parts that are not matrix products:
//   * the router's choice: softmax over the router's outputs, the `top` largest of (score + correction) are
//     chosen, their weights are the scores themselves (not renormalised).  The last outputs may stand for
//     experts that are the identity.  The result is dense: gates [T, experts] (zero where an expert was not
//     chosen) and, per token, the sum of the chosen identity experts' scores.
//   * the experts' activation with the gate folded in: act[t, e*ff + c] = act(u[t, e*ff + c]) * gates[t, e]
//     (squared relu), so that ONE product with the experts' down matrices side by side gives the weighted sum of
//     the chosen experts - an expert that was not chosen contributes exact zeros.
//   * dst[t,:] (+)= a[t] * src[t,:], the identity experts' share.
// All arithmetic is 32-bit.  A token's result depends on its own row only.
#include "common.cuh"

#define ROUTE_WARPS 4

// z [T, n] float router outputs; corr [n] float (null: none); gates [T, E] float; ident [T] float (null if n == E)
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ z, const float* __restrict__ corr, float* __restrict__ gates,
                 float* __restrict__ ident, int T, int n, int E, int top) {
    extern __shared__ float sm[];                              // per warp: scores [n], choice [n]
    pdl_trigger(); pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;                                        // no block-wide barrier below
    float* score = sm + (size_t)warp * 2 * n;
    float* choice = score + n;
    const float* zr = z + (size_t)t * n;
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, zr[i]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int i = lane; i < n; i += 32) { const float e = expf(zr[i] - m); score[i] = e; sum += e; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int i = lane; i < n; i += 32) {
        const float s = score[i] * inv;
        score[i] = s;
        choice[i] = s + (corr ? corr[i] : 0.0f);
    }
    for (int i = lane; i < E; i += 32) gates[(size_t)t * E + i] = 0.0f;
    __syncwarp();
    float idw = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float c = choice[i];
            if (c > best) { best = c; at = i; }                // ascending i: the first of equal values
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= n) break;                                    // fewer outputs than `top` (or nothing comparable left)
        if (lane == 0) {
            choice[at] = -INFINITY;
            if (at < E) gates[(size_t)t * E + at] = score[at];
        }
        if (at >= E) idw += score[at];
        __syncwarp();
    }
    if (ident && lane == 0) ident[t] = idw;
}

extern "C" int rb_moe_route(const float* z, const float* corr, float* gates, float* ident, int T, int n, int E, int top,
                            void* stream) {
    if (T <= 0) return 0;
    if (n <= 0 || E < 0 || E > n || top <= 0 || top > n) RB_REFUSE("moe_route: %d outputs, %d experts, top %d", n, E, top);
    if (n > E && !ident) RB_REFUSE("moe_route: identity experts need a place for their weights");
    const size_t smem = (size_t)ROUTE_WARPS * 2 * n * sizeof(float);
    if (smem > 48 * 1024) RB_REFUSE("moe_route: %d router outputs", n);
    return rb_launch(moe_route_kernel, dim3(rb_ceil_div(T, ROUTE_WARPS)), dim3(ROUTE_WARPS * 32), smem, (cudaStream_t)stream,
                     z, corr, gates, ident, T, n, E, top);
}

// act[t, c] = relu(u[t, c])^2 * gates[t, c / ff]
template <typename TA>
__global__ void relu2_gate_kernel(const TA* __restrict__ u, const float* __restrict__ gates, TA* __restrict__ act,
                                  int T, int E, int ff) {
    pdl_trigger(); pdl_wait();
    const int width = E * ff;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float g = gates[(size_t)t * E + c / ff];
        float v = 0.0f;
        if (g != 0.0f) {
            const float r = fmaxf(to_f32(u[(size_t)t * width + c]), 0.0f);
            v = r * r * g;
        }
        act[(size_t)t * width + c] = from_f32<TA>(v);
    }
}

extern "C" int rb_relu2_gate(const void* u, const float* gates, void* act, int dtype, int T, int E, int ff, void* stream) {
    if (T <= 0 || E <= 0) return 0;
    if (ff <= 0) RB_REFUSE("relu2_gate: inner width %d", ff);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(rb_ceil_div((long long)E * ff, 256), T < 65535 ? T : 65535);
    if (dtype == RB_F32) return rb_launch(relu2_gate_kernel<float>, grid, dim3(256), 0, s, (const float*)u, gates, (float*)act, T, E, ff);
    if (dtype == RB_BF16) return rb_launch(relu2_gate_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)u, gates, (bf16*)act, T, E, ff);
    RB_REFUSE("relu2_gate: dtype %d", dtype);
}

// dst[t,:] = a[t] * src[t,:] (store) or dst[t,:] += a[t] * src[t,:]
template <typename TS>
__global__ void rows_axpy_kernel(float* __restrict__ dst, const float* __restrict__ a, const TS* __restrict__ src, int T, int h, int store) {
    pdl_trigger(); pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= h) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float v = a[t] * to_f32(src[(size_t)t * h + c]);
        float* d = dst + (size_t)t * h + c;
        *d = store ? v : *d + v;
    }
}

extern "C" int rb_rows_axpy(float* dst, const float* a, const void* src, int src_dtype, int T, int h, int store, void* stream) {
    if (T <= 0 || h <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(rb_ceil_div(h, 256), T < 65535 ? T : 65535);
    if (src_dtype == RB_F32) return rb_launch(rows_axpy_kernel<float>, grid, dim3(256), 0, s, dst, a, (const float*)src, T, h, store);
    if (src_dtype == RB_BF16) return rb_launch(rows_axpy_kernel<bf16>, grid, dim3(256), 0, s, dst, a, (const bf16*)src, T, h, store);
    RB_REFUSE("rows_axpy: dtype %d", src_dtype);
}
