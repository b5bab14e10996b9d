// Linear recurrences over a matrix state per (request, head), token by token:
//
//   S [dk, dv] float, rows = key channels, one per request slot and head, carried from step to step.
//   form 0 (diagonal gate):        S <- diag(g) S + k v^T                              o = S^T q
//   form 1 (delta, old state):     S <- diag(g) S - (a*u)(u^T S_old) + k v^T           o = S^T q      u = k / |k|
//   form 2 (delta, gated state):   S <- diag(g) S;  S <- S + k (beta (v - S^T k))^T    o = S^T q
//
// A column of S (one value channel) evolves on its own, so the work is split by columns: a CTA owns
// RR_COLS columns of one (request, head), a column is shared by RR_SPLIT adjacent lanes that hold RP rows
// each in registers, and the two dot products per token are completed by two shuffles in a fixed order.
// The CTA walks its request's tokens of this step in order; per tile of tokens all threads first prepare
// the token vectors in shared memory - the gate from its pre-activation, unit vectors, scales - in float:
// (a gate is held as g - 1 = expm1(ln g) and applied as S + (g - 1) S, so that a gate near 1 keeps its digits)
//   gate 0:  g = sigmoid(z)^(1/tau)                 = exp(-softplus(-z) / tau)
//   gate 1:  g = exp(-c * sigmoid(z))
//   gate 2:  g = exp(-exp(rate[h]) * softplus(z))
// Everything that enters the recurrence besides the projections is 32-bit; the sequence of operations for
// a token does not depend on how the request was cut into steps or on the batch.
#include "common.cuh"

#define RR_THREADS 128
#define RR_COLS 32
#define RR_SPLIT 4

struct RecurArgs {
    const void* q; long long ldq;          // [T, Hk * dk]   (activation dtype)
    const void* k; long long ldk;          // [T, Hk * dk]
    const void* v; long long ldv;          // [T, H * dv]
    const float* z; long long ldz;         // [T, H * dk] gate pre-activation without its bias
    const float* z_bias;                   // [H * dk] or null
    const void* a_pre; long long lda;      // form 1: removal rate before the sigmoid [T, H * dk] (activation dtype)
    const float* a_bias;                   // form 1: [H * dk] or null
    const void* b_pre; long long ldb;      // form 2: write strength before the sigmoid [T, H]
    const float* rate;                     // gate 2: [H]
    float gate_param;                      // gate 0: 1 / tau;  gate 1: c
    float q_scale;                         // q is multiplied by this (after it was made a unit vector, if it is)
    int unit_qk;                           // q and k are made unit vectors: x / sqrt(sum x^2 + 1e-6)
    int gate;
    float* state;                          // [slots, H, dk, dv]
    float* out;                            // [T, H, dv]
    const int* cu_q; const int* entry_slot;
    int H, Hk, dk, dv, tile;
};

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename TA, int FORM, int RP>
__global__ void __launch_bounds__(RR_THREADS)
recurrence_kernel(const RecurArgs A) {
    constexpr int RPP = RP + 4;                       // row slices of the RR_SPLIT lanes lie in different banks
    constexpr int VEC = RR_SPLIT * RPP;
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, e = blockIdx.z;
    const int c0 = blockIdx.x * RR_COLS;
    const int kvh = h / (A.H / A.Hk);
    const int dk = A.dk, dv = A.dv, TT = A.tile;
    float* qs = sm;
    float* ks = qs + TT * VEC;
    float* gs = ks + TT * VEC;
    float* us = gs + TT * VEC;                        // form 1 only
    float* as = us + (FORM == 1 ? TT * VEC : 0);      // form 1 only
    float* vs = as + (FORM == 1 ? TT * VEC : 0);
    float* bs = vs + TT * RR_COLS;
    const float rate = (A.gate == 2) ? expf(A.rate[h]) : 0.0f;     // weights: read before the wait
    pdl_wait();
    const int s0 = A.cu_q[e], n = A.cu_q[e + 1] - s0;
    const int slot = A.entry_slot[e];
    const int cl = warp * (32 / RR_SPLIT) + lane / RR_SPLIT;       // column of this thread inside the CTA's block
    const int r = lane % RR_SPLIT;
    const int c = c0 + cl;
    float* S = A.state + ((size_t)slot * A.H + h) * dk * dv;
    float s[RP];
#pragma unroll
    for (int ii = 0; ii < RP; ++ii) {
        const int i = r * RP + ii;
        s[ii] = (i < dk && c < dv) ? S[(size_t)i * dv + c] : 0.0f;
    }
    const TA* q = (const TA*)A.q; const TA* k = (const TA*)A.k; const TA* v = (const TA*)A.v;
    for (int base = 0; base < n; base += TT) {
        const int nt = min(TT, n - base);
        __syncthreads();                               // the tile before has been read by everybody
        // ---- prepare the tile's token vectors
        for (int tt = warp; tt < nt; tt += RR_THREADS / 32) {
            const size_t t = (size_t)(s0 + base + tt);
            const TA* qr = q + t * A.ldq + (size_t)kvh * dk;
            const TA* kr = k + t * A.ldk + (size_t)kvh * dk;
            float qn = A.q_scale, kn = 1.0f, un = 1.0f;
            if (A.unit_qk || FORM == 1) {
                float sq = 0.0f, sk = 0.0f;
                for (int i = lane; i < dk; i += 32) {
                    const float a = to_f32(qr[i]), b = to_f32(kr[i]);
                    sq = fmaf(a, a, sq); sk = fmaf(b, b, sk);
                }
                sq = warp_sum(sq); sk = warp_sum(sk);
                if (A.unit_qk) { qn = A.q_scale / sqrtf(sq + 1e-6f); kn = 1.0f / sqrtf(sk + 1e-6f); }
                un = 1.0f / sqrtf(sk + 1e-6f);
            }
            for (int i = lane; i < RR_SPLIT * RP; i += 32) {
                const int at = tt * VEC + (i / RP) * RPP + (i % RP);
                float qv = 0.0f, kv = 0.0f, g = -1.0f, uv = 0.0f, av = 0.0f;
                if (i < dk) {
                    qv = to_f32(qr[i]) * qn;
                    const float kraw = to_f32(kr[i]);
                    kv = kraw * kn;
                    float z = A.z[t * A.ldz + (size_t)h * dk + i];
                    if (A.z_bias) z += A.z_bias[(size_t)h * dk + i];
                    // the gate is kept as g - 1 = expm1(ln g): a gate close to 1 (a memory that lasts thousands of
                    // tokens) then keeps the digits of 1 - g that rounding g itself to float would drop
                    float lg;
                    if (A.gate == 0) lg = -softplus_f(-z) * A.gate_param;
                    else if (A.gate == 1) lg = -A.gate_param * sigmoid_f(z);
                    else lg = -rate * softplus_f(z);
                    g = expm1f(lg);
                    if (FORM == 1) {
                        float ap = to_f32(((const TA*)A.a_pre)[t * A.lda + (size_t)h * dk + i]);
                        if (A.a_bias) ap += A.a_bias[(size_t)h * dk + i];
                        uv = kraw * un;
                        av = sigmoid_f(ap) * uv;
                    }
                }
                qs[at] = qv; ks[at] = kv; gs[at] = g;
                if (FORM == 1) { us[at] = uv; as[at] = av; }
            }
            {
                const int cc = c0 + lane;                  // RR_COLS == 32: a lane per column
                vs[tt * RR_COLS + lane] = cc < dv ? to_f32(v[t * A.ldv + (size_t)h * dv + cc]) : 0.0f;
            }
            if (FORM == 2 && lane == 0) bs[tt] = sigmoid_f(to_f32(((const TA*)A.b_pre)[t * A.ldb + h]));
        }
        __syncthreads();
        // ---- walk the tile
        for (int tt = 0; tt < nt; ++tt) {
            const float4* q4 = (const float4*)(qs + tt * VEC + r * RPP);
            const float4* k4 = (const float4*)(ks + tt * VEC + r * RPP);
            const float4* g4 = (const float4*)(gs + tt * VEC + r * RPP);
            const float vc = vs[tt * RR_COLS + cl];
            float o = 0.0f;
            if (FORM == 0) {
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 qq = q4[j], kk = k4[j], gg = g4[j];
                    s[4 * j + 0] = fmaf(gg.x, s[4 * j + 0], fmaf(kk.x, vc, s[4 * j + 0])); o = fmaf(s[4 * j + 0], qq.x, o);
                    s[4 * j + 1] = fmaf(gg.y, s[4 * j + 1], fmaf(kk.y, vc, s[4 * j + 1])); o = fmaf(s[4 * j + 1], qq.y, o);
                    s[4 * j + 2] = fmaf(gg.z, s[4 * j + 2], fmaf(kk.z, vc, s[4 * j + 2])); o = fmaf(s[4 * j + 2], qq.z, o);
                    s[4 * j + 3] = fmaf(gg.w, s[4 * j + 3], fmaf(kk.w, vc, s[4 * j + 3])); o = fmaf(s[4 * j + 3], qq.w, o);
                }
            } else if (FORM == 1) {
                const float4* u4 = (const float4*)(us + tt * VEC + r * RPP);
                const float4* a4 = (const float4*)(as + tt * VEC + r * RPP);
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 uu = u4[j];
                    dot = fmaf(uu.x, s[4 * j + 0], dot); dot = fmaf(uu.y, s[4 * j + 1], dot);
                    dot = fmaf(uu.z, s[4 * j + 2], dot); dot = fmaf(uu.w, s[4 * j + 3], dot);
                }
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 qq = q4[j], kk = k4[j], gg = g4[j], aa = a4[j];
                    s[4 * j + 0] = fmaf(gg.x, s[4 * j + 0], s[4 * j + 0] + fmaf(-aa.x, dot, kk.x * vc)); o = fmaf(s[4 * j + 0], qq.x, o);
                    s[4 * j + 1] = fmaf(gg.y, s[4 * j + 1], s[4 * j + 1] + fmaf(-aa.y, dot, kk.y * vc)); o = fmaf(s[4 * j + 1], qq.y, o);
                    s[4 * j + 2] = fmaf(gg.z, s[4 * j + 2], s[4 * j + 2] + fmaf(-aa.z, dot, kk.z * vc)); o = fmaf(s[4 * j + 2], qq.z, o);
                    s[4 * j + 3] = fmaf(gg.w, s[4 * j + 3], s[4 * j + 3] + fmaf(-aa.w, dot, kk.w * vc)); o = fmaf(s[4 * j + 3], qq.w, o);
                }
            } else {
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 kk = k4[j], gg = g4[j];
                    s[4 * j + 0] = fmaf(gg.x, s[4 * j + 0], s[4 * j + 0]); dot = fmaf(kk.x, s[4 * j + 0], dot);
                    s[4 * j + 1] = fmaf(gg.y, s[4 * j + 1], s[4 * j + 1]); dot = fmaf(kk.y, s[4 * j + 1], dot);
                    s[4 * j + 2] = fmaf(gg.z, s[4 * j + 2], s[4 * j + 2]); dot = fmaf(kk.z, s[4 * j + 2], dot);
                    s[4 * j + 3] = fmaf(gg.w, s[4 * j + 3], s[4 * j + 3]); dot = fmaf(kk.w, s[4 * j + 3], dot);
                }
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                const float dl = bs[tt] * (vc - dot);
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 qq = q4[j], kk = k4[j];
                    s[4 * j + 0] = fmaf(kk.x, dl, s[4 * j + 0]); o = fmaf(s[4 * j + 0], qq.x, o);
                    s[4 * j + 1] = fmaf(kk.y, dl, s[4 * j + 1]); o = fmaf(s[4 * j + 1], qq.y, o);
                    s[4 * j + 2] = fmaf(kk.z, dl, s[4 * j + 2]); o = fmaf(s[4 * j + 2], qq.z, o);
                    s[4 * j + 3] = fmaf(kk.w, dl, s[4 * j + 3]); o = fmaf(s[4 * j + 3], qq.w, o);
                }
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (r == 0 && c < dv) A.out[((size_t)(s0 + base + tt) * A.H + h) * dv + c] = o;
        }
    }
#pragma unroll
    for (int ii = 0; ii < RP; ++ii) {
        const int i = r * RP + ii;
        if (i < dk && c < dv) S[(size_t)i * dv + c] = s[ii];
    }
}

template <typename TA, int FORM>
static int recurrence_launch_rp(const RecurArgs& A, int n_entries, cudaStream_t st) {
    RecurArgs a = A;
    const int need = rb_ceil_div(a.dk, RR_SPLIT);
    const int rp = need <= 8 ? 8 : need <= 16 ? 16 : need <= 32 ? 32 : 64;
    a.tile = rp >= 64 ? 8 : 16;
    const int narr = FORM == 1 ? 5 : 3;
    const size_t smem = ((size_t)a.tile * (narr * RR_SPLIT * (rp + 4) + RR_COLS) + a.tile) * sizeof(float);
    dim3 grid(rb_ceil_div(a.dv, RR_COLS), a.H, n_entries);
    if (rp == 8) return rb_launch(recurrence_kernel<TA, FORM, 8>, grid, dim3(RR_THREADS), smem, st, a);
    if (rp == 16) return rb_launch(recurrence_kernel<TA, FORM, 16>, grid, dim3(RR_THREADS), smem, st, a);
    if (rp == 32) return rb_launch(recurrence_kernel<TA, FORM, 32>, grid, dim3(RR_THREADS), smem, st, a);
    return rb_launch(recurrence_kernel<TA, FORM, 64>, grid, dim3(RR_THREADS), smem, st, a);
}

// form: 0, 1, 2 as above.  All row strides in elements.  state [slots, H, dk, dv] float; out [T, H, dv] float.
extern "C" int rb_recurrence(int form, int gate, int dtype,
                             const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                             const float* z, long long ldz, const float* z_bias,
                             const void* a_pre, long long lda, const float* a_bias,
                             const void* b_pre, long long ldb, const float* rate,
                             float gate_param, float q_scale, int unit_qk,
                             float* state, float* out, const int* cu_q, const int* entry_slot,
                             int n_entries, int H, int Hk, int dk, int dv, void* stream) {
    if (n_entries <= 0) return 0;
    if (H <= 0 || Hk <= 0 || H % Hk) RB_REFUSE("recurrence: %d heads over %d key heads", H, Hk);
    if (dk <= 0 || dk > 64 * RR_SPLIT || dv <= 0) RB_REFUSE("recurrence: key size %d (1..%d), value size %d", dk, 64 * RR_SPLIT, dv);
    if (form < 0 || form > 2 || gate < 0 || gate > 2) RB_REFUSE("recurrence: form %d, gate %d", form, gate);
    if (form == 1 && !a_pre) RB_REFUSE("recurrence: the delta form on the old state needs removal rates");
    if (form == 2 && !b_pre) RB_REFUSE("recurrence: the gated delta form needs write strengths");
    if (gate == 2 && !rate) RB_REFUSE("recurrence: gate 2 needs a rate per head");
    if (n_entries > 65535 || H > 65535) RB_REFUSE("recurrence: %d requests, %d heads exceed the grid", n_entries, H);
    RecurArgs A;
    A.q = q; A.ldq = ldq; A.k = k; A.ldk = ldk; A.v = v; A.ldv = ldv; A.z = z; A.ldz = ldz; A.z_bias = z_bias;
    A.a_pre = a_pre; A.lda = lda; A.a_bias = a_bias; A.b_pre = b_pre; A.ldb = ldb; A.rate = rate;
    A.gate_param = gate_param; A.q_scale = q_scale; A.unit_qk = unit_qk; A.gate = gate;
    A.state = state; A.out = out; A.cu_q = cu_q; A.entry_slot = entry_slot;
    A.H = H; A.Hk = Hk; A.dk = dk; A.dv = dv; A.tile = 16;
    cudaStream_t st = (cudaStream_t)stream;
#define RB_RECUR(TA) \
    do { if (form == 0) return recurrence_launch_rp<TA, 0>(A, n_entries, st); \
         if (form == 1) return recurrence_launch_rp<TA, 1>(A, n_entries, st); \
         return recurrence_launch_rp<TA, 2>(A, n_entries, st); } while (0)
    if (dtype == RB_F32) RB_RECUR(float);
    if (dtype == RB_BF16) RB_RECUR(bf16);
#undef RB_RECUR
    RB_REFUSE("recurrence: dtype %d", dtype);
}
