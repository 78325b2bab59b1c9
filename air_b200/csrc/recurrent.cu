// Mixers that carry a state of fixed size from token to token, over the step's flat batch: every entry of the
// batch brings the next tokens of one request (a portion of a prompt or one decoded token), rows
// q_start[e] .. q_start[e + 1] of the step, and slots[e] is the request's row of the state tensors (negative:
// padding, skipped).  Everything here is 32-bit: inputs, states and arithmetic.
//
//   short_conv_silu_kernel   y[t, c] = silu(sum_j w[c, j] x[t - (taps - 1 - j), c]): a causal convolution over time
//                            per channel whose last taps - 1 inputs are the state (zeros before a request's start)
//   linear_scan_kernel       a state S [d, dv] per head, updated token by token, read out after each update:
//                              DELTA  S = g S;  u = beta (v - S^T k);  S += k u^T;  o = S^T q   (one decay per head)
//                              GLA    S = diag(alpha) S + k v^T;  o = S^T q                      (a decay per key channel)
//                            Columns of S do not depend on one another, so a block takes a few of them and a column is
//                            held in the registers of L lanes of one warp; the tokens of a portion are taken in order.
//                            What a token's output is depends on the state and the tokens before it only, not on how
//                            the request was cut into steps or on the rest of the batch.
//   gated_rmsnorm_kernel     out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :])
#include "common.cuh"

namespace air {

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_THREADS = 128;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// x [T, ld] (the first C columns), w [C, taps], state [slots, C, taps - 1] (oldest first), y [T, C].
// grid (channel blocks, entries, chunks of `chunk` tokens); the thread of a channel in the first chunk of an
// entry is the only one that reads or writes the channel's state.
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_silu_kernel(const float* __restrict__ x, int ld, const float* __restrict__ w, float* __restrict__ state,
                       float* __restrict__ y, const int* __restrict__ q_start, const int* __restrict__ slots,
                       int C, int taps, int chunk) {
    pdl_enter(TR_CONV);
    const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
    const int e = blockIdx.y;
    const int slot = slots[e];
    if (c >= C || slot < 0) return;
    const int q0 = q_start[e], n = q_start[e + 1] - q0;
    const int t0 = blockIdx.z * chunk;
    if (t0 >= n && blockIdx.z > 0) return;
    const int t1 = min(n, t0 + chunk);
    const int keep = taps - 1;
    float wv[CONV_MAX_TAPS], win[CONV_MAX_TAPS], old[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        wv[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        win[j] = 0.f;
        old[j] = 0.f;
    }
    float* st = state + ((size_t)slot * C + c) * keep;
    // win[i]: the input (taps - 1 - i) tokens before the next one
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
        if (i < keep) {
            const int idx = t0 - keep + i;
            win[i] = idx >= 0 ? x[(size_t)(q0 + idx) * ld + c] : st[keep + idx];
            old[i] = win[i];
        }
    }
    for (int t = t0; t < t1; ++t) {
        const float cur = x[(size_t)(q0 + t) * ld + c];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
            if (i < keep) acc = fmaf(wv[i], win[i], acc);
        acc = fmaf(wv[keep], cur, acc);
        y[(size_t)(q0 + t) * C + c] = silu_f(acc);
#pragma unroll
        for (int i = 0; i < CONV_MAX_TAPS - 2; ++i)
            if (i + 1 < keep) win[i] = win[i + 1];
        if (keep > 0) win[keep - 1] = cur;
    }
    if (blockIdx.z == 0) {
        // the state after the portion: its last taps - 1 inputs, or older ones from the state as it was
#pragma unroll
        for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
            if (i < keep) {
                const int idx = n - keep + i;
                st[i] = idx >= 0 ? x[(size_t)(q0 + idx) * ld + c] : old[i + n];
            }
        }
    }
}

enum { SCAN_DELTA = 0, SCAN_GLA = 1 };
constexpr int SCAN_THREADS = 128;
constexpr int SCAN_TOKENS = 16;      // tokens staged in shared memory at a time

struct ScanArgs {
    const float* q; int ldq;         // [T, ldq]: head g's d elements at column g * d
    const float* k; int ldk;
    const float* v; int ldv;         // head h's dv elements at column h * dv
    const float* decay; int ldd;     // DELTA: [T, ldd] one logit per head;  GLA: [T, ldd] d logits per head
    const float* beta; int ldb;      // DELTA: [T, ldb] one logit per head
    const float* a_log;              // DELTA: [H]
    const float* dt_bias;            // DELTA: [H]
    float* state;                    // [slots, H, d, dv]
    float* out;                      // [T, H, dv]
    const int* q_start;
    const int* slots;
    int H, G, d, dv, L;              // G: heads of q and k (head h reads h / (H / G)); L lanes hold a column
    float q_scale, inv_tau, unit_eps;
    int unit;                        // q and k are divided by sqrt(sum of squares + unit_eps) first
};

template <int MODE, int R>
__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(const ScanArgs p) {
    extern __shared__ float smem[];
    pdl_enter(TR_SCAN);
    const int L = p.L, cpw = 32 / L, CB = SCAN_THREADS / L, dpad = L * R;
    const int e = blockIdx.z, h = blockIdx.y;
    const int slot = p.slots[e];
    if (slot < 0) return;
    const int q0 = p.q_start[e], n = p.q_start[e + 1] - q0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane / cpw;                                    // which rows of the column: l, l + L, l + 2L, ...
    const int cc = warp * cpw + lane % cpw;                      // column within the block
    const int col = blockIdx.x * CB + cc;
    const bool live = col < p.dv;
    const int g = h / (p.H / p.G);

    float* sk = smem;                                            // [SCAN_TOKENS][dpad]
    float* sq = sk + SCAN_TOKENS * dpad;                         // [SCAN_TOKENS][dpad]
    float* sa = sq + SCAN_TOKENS * dpad;                         // GLA: [SCAN_TOKENS][dpad];  DELTA: g, beta [2][SCAN_TOKENS]
    float* sv = sa + (MODE == SCAN_GLA ? SCAN_TOKENS * dpad : 2 * SCAN_TOKENS);   // [SCAN_TOKENS][CB]
    float* so = sv + SCAN_TOKENS * CB;                           // [SCAN_TOKENS][CB]

    float S[R];
    float* st = p.state + ((size_t)slot * p.H + h) * p.d * p.dv;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = i * L + l;
        S[i] = (live && r < p.d) ? st[(size_t)r * p.dv + col] : 0.f;
    }
    float neg_a = 0.f, dtb = 0.f;
    if (MODE == SCAN_DELTA) {
        neg_a = -expf(p.a_log[h]);
        dtb = p.dt_bias[h];
    }

    for (int t0 = 0; t0 < n; t0 += SCAN_TOKENS) {
        const int cnt = min(SCAN_TOKENS, n - t0);
        for (int idx = threadIdx.x; idx < SCAN_TOKENS * dpad; idx += SCAN_THREADS) {
            const int tt = idx / dpad, r = idx % dpad;
            float kv = 0.f, qv = 0.f, av = 1.f;
            if (tt < cnt && r < p.d) {
                const size_t row = (size_t)(q0 + t0 + tt);
                kv = p.k[row * p.ldk + g * p.d + r];
                qv = p.q[row * p.ldq + g * p.d + r];
                if (MODE == SCAN_GLA) {
                    qv *= p.q_scale;
                    av = expf(p.inv_tau * log_sigmoid_f(p.decay[row * p.ldd + h * p.d + r]));
                }
            }
            sk[idx] = kv;
            sq[idx] = qv;
            if (MODE == SCAN_GLA) sa[idx] = av;
        }
        for (int idx = threadIdx.x; idx < SCAN_TOKENS * CB; idx += SCAN_THREADS) {
            const int tt = idx / CB, c = blockIdx.x * CB + idx % CB;
            sv[idx] = (tt < cnt && c < p.dv) ? p.v[(size_t)(q0 + t0 + tt) * p.ldv + h * p.dv + c] : 0.f;
        }
        if (MODE == SCAN_DELTA && threadIdx.x < SCAN_TOKENS) {
            const int tt = threadIdx.x;
            float gv = 1.f, bv = 0.f;
            if (tt < cnt) {
                const size_t row = (size_t)(q0 + t0 + tt);
                gv = expf(neg_a * softplus_f(p.decay[row * p.ldd + h] + dtb));
                bv = 1.f / (1.f + expf(-p.beta[row * p.ldb + h]));
            }
            sa[tt] = gv;
            sa[SCAN_TOKENS + tt] = bv;
        }
        __syncthreads();
        if (p.unit) {
            // q and k of every staged token to unit length (q also times q_scale): a warp per vector
            for (int item = warp; item < 2 * cnt; item += SCAN_THREADS / 32) {
                float* vec = (item & 1 ? sq : sk) + (item >> 1) * dpad;
                float ss = 0.f;
                for (int r = lane; r < p.d; r += 32) ss = fmaf(vec[r], vec[r], ss);
                ss = warp_sum(ss);
                const float f = (item & 1 ? p.q_scale : 1.f) / sqrtf(ss + p.unit_eps);
                for (int r = lane; r < p.d; r += 32) vec[r] *= f;
            }
            __syncthreads();
        }
        for (int tt = 0; tt < cnt; ++tt) {
            const float* kk = sk + tt * dpad + l;
            const float* qq = sq + tt * dpad + l;
            const float vv = sv[tt * CB + cc];
            float o = 0.f;
            if (MODE == SCAN_DELTA) {
                const float gv = sa[tt], bv = sa[SCAN_TOKENS + tt];
                float pred = 0.f;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] *= gv;
                    pred = fmaf(S[i], kk[i * L], pred);
                }
                for (int off = 16; off >= cpw; off >>= 1) pred += __shfl_xor_sync(0xffffffffu, pred, off);
                const float u = bv * (vv - pred);
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] = fmaf(kk[i * L], u, S[i]);
                    o = fmaf(S[i], qq[i * L], o);
                }
            } else {
                const float* aa = sa + tt * dpad + l;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[i] = fmaf(aa[i * L], S[i], kk[i * L] * vv);
                    o = fmaf(S[i], qq[i * L], o);
                }
            }
            for (int off = 16; off >= cpw; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
            if (l == 0) so[tt * CB + cc] = o;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < cnt * CB; idx += SCAN_THREADS) {
            const int tt = idx / CB, c = blockIdx.x * CB + idx % CB;
            if (c < p.dv) p.out[((size_t)(q0 + t0 + tt) * p.H + h) * p.dv + c] = so[idx];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int r = i * L + l;
        if (live && r < p.d) st[(size_t)r * p.dv + col] = S[i];
    }
}

// o [T, H, dv] float32; gate [T, ldg] float32 (head h at column h * dv); w [dv]; out [T, H * dv].
// One warp per (token, head).
template <typename TO>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int ldg, const float* __restrict__ w,
                     TO* __restrict__ out, const int* __restrict__ token_seq, int T, int H, int dv, float eps) {
    pdl_enter(TR_GATED);
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * H) return;
    const int t = item / H, h = item % H;
    if (token_seq[t] < 0) return;
    const float* row = o + (size_t)item * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)dv + eps);
    const float* gr = gate + (size_t)t * ldg + h * dv;
    for (int i = lane; i < dv; i += 32)
        out[(size_t)item * dv + i] = from_float<TO>(row[i] * scale * w[i] * silu_f(gr[i]));
}

template <int MODE>
static int launch_scan(const ScanArgs& a, int S, cudaStream_t stream) {
    // rows of a column per lane: 16 up to 512 key channels, 32 beyond; lanes per column: the power of two that covers d
    const int R = a.d <= 512 ? 16 : 32;
    int L = 1;
    while (L * R < a.d) L *= 2;
    if (L > 32) return AIR_ERR_BAD_ARGUMENT;
    ScanArgs p = a;
    p.L = L;
    const int CB = SCAN_THREADS / L, dpad = L * R;
    const size_t smem = sizeof(float) * ((size_t)SCAN_TOKENS * dpad * (MODE == SCAN_GLA ? 3 : 2) +
                                         (MODE == SCAN_GLA ? 0 : 2 * SCAN_TOKENS) + 2 * (size_t)SCAN_TOKENS * CB);
    dim3 grid((a.dv + CB - 1) / CB, a.H, S);
    if (a.H > 65535 || S > 65535) return AIR_ERR_BAD_ARGUMENT;
    if (R == 16) {
        auto kernel = linear_scan_kernel<MODE, 16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch(kernel, grid, SCAN_THREADS, smem, stream, p);
    }
    auto kernel = linear_scan_kernel<MODE, 32>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch(kernel, grid, SCAN_THREADS, smem, stream, p);
}

}  // namespace air

AIR_API int air_short_conv_silu(const float* x, int ld, const float* w, float* state, float* y, const int* q_start,
                                const int* slots, int S, int C, int taps, int max_tokens, cudaStream_t stream) {
    if (S <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > air::CONV_MAX_TAPS || S > 65535) return AIR_ERR_BAD_ARGUMENT;
    const int chunk = 64;
    int chunks = (max_tokens + chunk - 1) / chunk;
    if (chunks < 1) chunks = 1;
    if (chunks > 65535) return AIR_ERR_BAD_ARGUMENT;
    dim3 grid((C + air::CONV_THREADS - 1) / air::CONV_THREADS, S, chunks);
    return air::launch(air::short_conv_silu_kernel, grid, air::CONV_THREADS, 0, stream, x, ld, w, state, y, q_start,
                       slots, C, taps, chunk);
}

AIR_API int air_linear_scan(int mode, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                            const float* decay, int ldd, const float* beta, int ldb, const float* a_log,
                            const float* dt_bias, float* state, float* out, const int* q_start, const int* slots,
                            int S, int H, int G, int d, int dv, float q_scale, float inv_tau, int unit, float unit_eps,
                            cudaStream_t stream) {
    if (S <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0) return AIR_ERR_BAD_ARGUMENT;
    air::ScanArgs a;
    a.q = q; a.ldq = ldq; a.k = k; a.ldk = ldk; a.v = v; a.ldv = ldv; a.decay = decay; a.ldd = ldd;
    a.beta = beta; a.ldb = ldb; a.a_log = a_log; a.dt_bias = dt_bias; a.state = state; a.out = out;
    a.q_start = q_start; a.slots = slots; a.H = H; a.G = G; a.d = d; a.dv = dv; a.L = 0;
    a.q_scale = q_scale; a.inv_tau = inv_tau; a.unit_eps = unit_eps; a.unit = unit;
    if (mode == air::SCAN_DELTA) return air::launch_scan<air::SCAN_DELTA>(a, S, stream);
    if (mode == air::SCAN_GLA) return air::launch_scan<air::SCAN_GLA>(a, S, stream);
    return AIR_ERR_BAD_ARGUMENT;
}

AIR_API int air_gated_rmsnorm(const float* o, const float* gate, int ldg, const float* w, void* out, int out_dtype,
                              const int* token_seq, int T, int H, int dv, float eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int blocks = (T * H + 3) / 4;
    AIR_DISPATCH(out_dtype, TO, return air::launch(air::gated_rmsnorm_kernel<TO>, blocks, 128, 0, stream, o, gate, ldg, w,
                                                   (TO*)out, token_seq, T, H, dv, eps));
    return 0;
}

AIR_API int air_trace_set_recurrent(unsigned long long* buffer) { return air::set_trace_here(buffer); }
