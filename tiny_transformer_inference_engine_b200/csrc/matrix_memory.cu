// Recurrent layers whose per-head state is a matrix S [key channels x value channels] that every token updates by a rank-one
// term: the RWKV-style time mix with a decay per key channel (wkv) and the xLSTM matrix memory with scalar gates and a running
// maximum (mlstm).  All of a recurrence is 32-bit: decays, gates, exponentials, the state and the read-out.
//
// Both scans share one layout.  A value column of S moves independently of the others, so a thread owns KPT consecutive key
// channels of one column: a CTA is (columns x slices) threads for one (request, head), slices = key channels / KPT rounded up
// to a power of two, the lanes of a column's slices adjacent so that the read-out sum over key channels is a few shuffles.
// The state rows hold S as [head][value column][padded key channels] (a thread's channels are contiguous).  The step's tokens
// of a request are walked in order, TB at a time staged through shared memory (decays and gates are evaluated while staging);
// a request may be cut into steps anywhere because the walk starts from the state row and ends by writing it back.
//
//   token_shift_mix   mixes[m][t] = h_t + (h_(t-1) - h_t) * mu[m]; the previous token of a step's first token is the state row
//   wkv_scan          o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T, w = exp(-exp(wlog + w0));
//                     also stores the request's last mixer input as the next step's previous token
//   mlstm_scan        i = cap tanh(i'/cap), f = logsigmoid(cap tanh(f'/cap)), m' = max(f + m, i), S <- e^(f+m-m') S + e^(i-m') k v^T,
//                     n likewise with k alone, o = S^T q / (max(|n.q|, e^(-m')) + 1e-6)
//   head_norm_gate    out = o / rms(o over the head) * weight * act(gate)   (act: silu or sigmoid)
#include "common.cuh"
#include <math.h>
using namespace ttie;

namespace {

constexpr int KPT = 16;          // key channels per thread
constexpr int TB = 16;           // tokens staged at a time

__device__ __forceinline__ int slot_row_(int slot, int num_rows) { return slot < 0 ? num_rows - 1 : slot; }

__device__ __forceinline__ float slice_sum(float v, int slices) {
    for (int o = 1; o < slices; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ x, long long ld, int T_, int d, int M, const float* __restrict__ mu,
                                       const float* __restrict__ prev, int prev_rows, const int* __restrict__ token_seq,
                                       const int* __restrict__ qsl, const int* __restrict__ slot_ids, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= d) return;
    for (int t = blockIdx.y; t < T_; t += gridDim.y) {
        const int s = token_seq[t];
        const float h = to_f32(x[(size_t)t * ld + c]);
        const float hp = t > qsl[s] ? to_f32(x[(size_t)(t - 1) * ld + c]) : prev[(size_t)slot_row_(slot_ids[s], prev_rows) * d + c];
        for (int m = 0; m < M; ++m)
            out[((size_t)m * T_ + t) * d + c] = from_f32<T>(fmaf(hp - h, mu[(size_t)m * d + c], h));
    }
}

struct WkvArgs {
    const void* r; const void* k; const void* v; long long ld;       // [T, H*D] each, compute dtype
    const float* wlog; long long ld_w; const float* w0; const float* u;
    float* state; int state_rows;                                     // [rows, H, D, Dpad]
    const void* x; long long ld_x; int d; float* prev; int prev_rows; // the mixer's input and the rows that keep its last token
    const int* qsl; const int* slot_ids;
    float* out;                                                       // [T, H*D] float32
    int H, D, Dpad, slices;
};

template <typename T>
__global__ void __launch_bounds__(128) wkv_scan_kernel(const WkvArgs a) {
    TTIE_PDL_ENTRY();
    extern __shared__ float sm[];
    const int cols = blockDim.x / a.slices;
    float* r_s = sm;                                                 // [TB][Dpad]
    float* k_s = r_s + TB * a.Dpad;
    float* w_s = k_s + TB * a.Dpad;
    float* v_s = w_s + TB * a.Dpad;                                  // [TB][cols]
    const int s = blockIdx.z, h = blockIdx.y;
    const int t0 = a.qsl[s], n = a.qsl[s + 1] - t0;
    const int slice = threadIdx.x % a.slices, cl = threadIdx.x / a.slices;
    const int col = blockIdx.x * cols + cl;
    const bool colv = col < a.D;
    const int HD = a.H * a.D;
    const size_t row = slot_row_(a.slot_ids[s], a.state_rows);
    float* sp = a.state + ((row * a.H + h) * a.D + (colv ? col : 0)) * a.Dpad + slice * KPT;
    float S[KPT], ub[KPT];
#pragma unroll
    for (int i = 0; i < KPT; i += 4) {
        const float4 x4 = colv ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[i] = x4.x; S[i + 1] = x4.y; S[i + 2] = x4.z; S[i + 3] = x4.w;
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) { const int ch = slice * KPT + i; ub[i] = ch < a.D ? a.u[h * a.D + ch] : 0.f; }
    const T* rp = reinterpret_cast<const T*>(a.r);
    const T* kp = reinterpret_cast<const T*>(a.k);
    const T* vp = reinterpret_cast<const T*>(a.v);
    for (int c0 = 0; c0 < n; c0 += TB) {
        const int nb = min(TB, n - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < nb * a.Dpad; e += blockDim.x) {
            const int tt = e / a.Dpad, ch = e - tt * a.Dpad;
            float rv = 0.f, kv = 0.f, wv = 0.f;
            if (ch < a.D) {
                const size_t g = (size_t)(t0 + c0 + tt);
                rv = to_f32(rp[g * a.ld + h * a.D + ch]);
                kv = to_f32(kp[g * a.ld + h * a.D + ch]);
                wv = expf(-expf(a.wlog[g * a.ld_w + h * a.D + ch] + a.w0[h * a.D + ch]));
            }
            r_s[e] = rv; k_s[e] = kv; w_s[e] = wv;
        }
        for (int e = threadIdx.x; e < nb * cols; e += blockDim.x) {
            const int tt = e / cols, c = blockIdx.x * cols + (e - tt * cols);
            v_s[e] = c < a.D ? to_f32(vp[(size_t)(t0 + c0 + tt) * a.ld + h * a.D + c]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float vj = v_s[tt * cols + cl];
            const float* rr = r_s + tt * a.Dpad + slice * KPT;
            const float* kk = k_s + tt * a.Dpad + slice * KPT;
            const float* ww = w_s + tt * a.Dpad + slice * KPT;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                const float kv = kk[i] * vj;
                acc = fmaf(rr[i], fmaf(ub[i], kv, S[i]), acc);
                S[i] = fmaf(ww[i], S[i], kv);
            }
            acc = slice_sum(acc, a.slices);
            if (slice == 0 && colv) a.out[(size_t)(t0 + c0 + tt) * HD + h * a.D + col] = acc;
        }
    }
    if (colv) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
    if (blockIdx.x == 0 && blockIdx.y == 0 && n > 0) {               // the request's last input is the next step's previous token
        const T* x = reinterpret_cast<const T*>(a.x) + (size_t)(t0 + n - 1) * a.ld_x;
        float* p = a.prev + (size_t)slot_row_(a.slot_ids[s], a.prev_rows) * a.d;
        for (int c = threadIdx.x; c < a.d; c += blockDim.x) p[c] = to_f32(x[c]);
    }
}

struct MlstmArgs {
    const void* q; const void* k; const void* v; long long ld;        // q, k [T, H*D]; v [T, H*Dv]; one row stride
    const float* gates; long long ld_g;                               // [T, 2H]: input gate pre-activations, then forget gate's
    float* S; float* nrm; float* mx; int state_rows;                  // [rows, H, Dv, Dpad], [rows, H, Dpad], [rows, H]
    const int* qsl; const int* slot_ids;
    float* out;                                                       // [T, H*Dv] float32
    int H, D, Dv, Dpad, slices; float qscale, cap;
};

__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T>
__global__ void __launch_bounds__(128) mlstm_scan_kernel(const MlstmArgs a) {
    TTIE_PDL_ENTRY();
    extern __shared__ float sm[];
    const int cols = blockDim.x / a.slices;
    float* q_s = sm;                                                 // [TB][Dpad]
    float* k_s = q_s + TB * a.Dpad;
    float* v_s = k_s + TB * a.Dpad;                                  // [TB][cols]
    float* g_s = v_s + TB * cols;                                    // [TB][3]: state decay, input weight, e^(-m)
    __shared__ float m_carry;
    const int s = blockIdx.z, h = blockIdx.y;
    const int t0 = a.qsl[s], n = a.qsl[s + 1] - t0;
    const int slice = threadIdx.x % a.slices, cl = threadIdx.x / a.slices;
    const int col = blockIdx.x * cols + cl;
    const bool colv = col < a.Dv;
    const size_t row = slot_row_(a.slot_ids[s], a.state_rows);
    float* sp = a.S + ((row * a.H + h) * a.Dv + (colv ? col : 0)) * a.Dpad + slice * KPT;
    float* np = a.nrm + (row * a.H + h) * a.Dpad + slice * KPT;
    float S[KPT], nv[KPT];
#pragma unroll
    for (int i = 0; i < KPT; i += 4) {
        const float4 x4 = colv ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[i] = x4.x; S[i + 1] = x4.y; S[i + 2] = x4.z; S[i + 3] = x4.w;
        const float4 n4 = *reinterpret_cast<const float4*>(np + i);
        nv[i] = n4.x; nv[i + 1] = n4.y; nv[i + 2] = n4.z; nv[i + 3] = n4.w;
    }
    if (threadIdx.x == 0) m_carry = a.mx[row * a.H + h];
    const T* qp = reinterpret_cast<const T*>(a.q);
    const T* kp = reinterpret_cast<const T*>(a.k);
    const T* vp = reinterpret_cast<const T*>(a.v);
    for (int c0 = 0; c0 < n; c0 += TB) {
        const int nb = min(TB, n - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < nb * a.Dpad; e += blockDim.x) {
            const int tt = e / a.Dpad, ch = e - tt * a.Dpad;
            float qv = 0.f, kv = 0.f;
            if (ch < a.D) {
                const size_t g = (size_t)(t0 + c0 + tt);
                qv = to_f32(qp[g * a.ld + h * a.D + ch]) * a.qscale;
                kv = to_f32(kp[g * a.ld + h * a.D + ch]);
            }
            q_s[e] = qv; k_s[e] = kv;
        }
        for (int e = threadIdx.x; e < nb * cols; e += blockDim.x) {
            const int tt = e / cols, c = blockIdx.x * cols + (e - tt * cols);
            v_s[e] = c < a.Dv ? to_f32(vp[(size_t)(t0 + c0 + tt) * a.ld + h * a.Dv + c]) : 0.f;
        }
        if (threadIdx.x == 0) {                                      // the gates' scalar recurrence over the staged tokens
            float m = m_carry;
            for (int tt = 0; tt < nb; ++tt) {
                const float* g = a.gates + (size_t)(t0 + c0 + tt) * a.ld_g;
                const float ig = a.cap * tanhf(g[h] / a.cap);
                const float fg = logsigmoidf_(a.cap * tanhf(g[a.H + h] / a.cap));
                const float m_new = fmaxf(fg + m, ig);
                g_s[3 * tt] = expf(fg + m - m_new);
                g_s[3 * tt + 1] = expf(ig - m_new);
                g_s[3 * tt + 2] = expf(-m_new);
                m = m_new;
            }
            m_carry = m;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float vj = v_s[tt * cols + cl];
            const float fa = g_s[3 * tt], ib = g_s[3 * tt + 1];
            const float* qq = q_s + tt * a.Dpad + slice * KPT;
            const float* kk = k_s + tt * a.Dpad + slice * KPT;
            float num = 0.f, nq = 0.f;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                const float bk = ib * kk[i];
                S[i] = fmaf(fa, S[i], bk * vj);
                nv[i] = fmaf(fa, nv[i], bk);
                num = fmaf(S[i], qq[i], num);
                nq = fmaf(nv[i], qq[i], nq);
            }
            num = slice_sum(num, a.slices);
            nq = slice_sum(nq, a.slices);
            if (slice == 0 && colv)
                a.out[(size_t)(t0 + c0 + tt) * a.H * a.Dv + h * a.Dv + col] = num / (fmaxf(fabsf(nq), g_s[3 * tt + 2]) + 1e-6f);
        }
    }
    if (colv) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
    if (blockIdx.x == 0 && cl == 0) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(np + i) = make_float4(nv[i], nv[i + 1], nv[i + 2], nv[i + 3]);
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) a.mx[row * a.H + h] = m_carry;
}

// one warp per (token, head)
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long ld_g, const float* __restrict__ w,
                                      int T_, int H, int Dv, float eps, int act, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)T_ * H) return;
    const long long t = unit / H;
    const int h = (int)(unit - t * H);
    const float* src = o + (size_t)unit * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) { const float v = src[j]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int j = lane; j < Dv; j += 32) {
        const float g = to_f32(gate[(size_t)t * ld_g + h * Dv + j]);
        const float sg = 1.0f / (1.0f + expf(-g));
        out[(size_t)unit * Dv + j] = from_f32<T>(src[j] * inv * w[h * Dv + j] * (act == 0 ? g * sg : sg));
    }
}

int scan_shape(int D, int cols_total, int units, int* slices, int* threads) {
    int sl = 1;
    while (sl * KPT < D) sl <<= 1;
    if (sl > 32) return -1;
    *slices = sl;
    // few (request, head) units: narrower CTAs so that the columns spread over more SMs
    int th = 128;
    while (th > 32 && (long long)units * ceil_div(cols_total, th / sl) < 2LL * num_sms()) th >>= 1;
    if (th < sl) th = sl < 32 ? 32 : sl;
    *threads = th;
    return 0;
}

}  // namespace

extern "C" int ttie_matrix_state_pad(int D) {                        // padded key channels of a state row
    int sl = 1;
    while (sl * KPT < D) sl <<= 1;
    return sl * KPT;
}

extern "C" int ttie_token_shift_mix(const void* x, long long ld, int T, int d, int M, const float* mu, const float* prev, int prev_rows,
                                    const int* token_seq, const int* qsl, const int* slot_ids, void* out, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(ceil_div(d, 256), T < 65535 ? T : 65535);
    if (dtype == kF32) TTIE_LAUNCH(token_shift_mix_kernel<float>, grid, 256, 0, s, (const float*)x, ld, T, d, M, mu, prev, prev_rows, token_seq, qsl, slot_ids, (float*)out);
    else if (dtype == kBF16) TTIE_LAUNCH(token_shift_mix_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)x, ld, T, d, M, mu, prev, prev_rows, token_seq, qsl, slot_ids, (__nv_bfloat16*)out);
    else TTIE_FAIL("token_shift_mix: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("token_shift_mix");
    return 0;
}

extern "C" int ttie_wkv_scan(const void* r, const void* k, const void* v, long long ld, const float* wlog, long long ld_w, const float* w0,
                             const float* u, float* state, int state_rows, const void* x, long long ld_x, int d, float* prev,
                             int prev_rows, const int* qsl, const int* slot_ids, int num_seqs, float* out, int H, int D, int dtype,
                             void* stream) {
    if (num_seqs <= 0) return 0;
    WkvArgs a;
    a.r = r; a.k = k; a.v = v; a.ld = ld; a.wlog = wlog; a.ld_w = ld_w; a.w0 = w0; a.u = u; a.state = state; a.state_rows = state_rows;
    a.x = x; a.ld_x = ld_x; a.d = d; a.prev = prev; a.prev_rows = prev_rows; a.qsl = qsl; a.slot_ids = slot_ids; a.out = out;
    a.H = H; a.D = D;
    int threads;
    if (scan_shape(D, D, num_seqs * H, &a.slices, &threads)) TTIE_FAIL("wkv_scan: %d key channels per head (at most %d)", D, 32 * KPT);
    a.Dpad = a.slices * KPT;
    const int cols = threads / a.slices;
    const size_t smem = (size_t)TB * (3 * a.Dpad + cols) * sizeof(float);
    dim3 grid(ceil_div(D, cols), H, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (smem > 48 * 1024) {                                          // (wide heads: more staging than a kernel gets unasked)
        cudaFuncSetAttribute(wkv_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(wkv_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (dtype == kF32) TTIE_LAUNCH(wkv_scan_kernel<float>, grid, threads, smem, s, a);
    else if (dtype == kBF16) TTIE_LAUNCH(wkv_scan_kernel<__nv_bfloat16>, grid, threads, smem, s, a);
    else TTIE_FAIL("wkv_scan: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("wkv_scan");
    return 0;
}

extern "C" int ttie_mlstm_scan(const void* q, const void* k, const void* v, long long ld, const float* gates, long long ld_g, float* S,
                               float* nrm, float* mx, int state_rows, const int* qsl, const int* slot_ids, int num_seqs, float* out,
                               int H, int D, int Dv, float qscale, float cap, int dtype, void* stream) {
    if (num_seqs <= 0) return 0;
    MlstmArgs a;
    a.q = q; a.k = k; a.v = v; a.ld = ld; a.gates = gates; a.ld_g = ld_g; a.S = S; a.nrm = nrm; a.mx = mx; a.state_rows = state_rows;
    a.qsl = qsl; a.slot_ids = slot_ids; a.out = out; a.H = H; a.D = D; a.Dv = Dv; a.qscale = qscale; a.cap = cap;
    int threads;
    if (scan_shape(D, Dv, num_seqs * H, &a.slices, &threads)) TTIE_FAIL("mlstm_scan: %d key channels per head (at most %d)", D, 32 * KPT);
    a.Dpad = a.slices * KPT;
    const int cols = threads / a.slices;
    const size_t smem = (size_t)TB * (2 * a.Dpad + cols + 3) * sizeof(float);
    dim3 grid(ceil_div(Dv, cols), H, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(mlstm_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(mlstm_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (dtype == kF32) TTIE_LAUNCH(mlstm_scan_kernel<float>, grid, threads, smem, s, a);
    else if (dtype == kBF16) TTIE_LAUNCH(mlstm_scan_kernel<__nv_bfloat16>, grid, threads, smem, s, a);
    else TTIE_FAIL("mlstm_scan: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("mlstm_scan");
    return 0;
}

extern "C" int ttie_head_norm_gate(const float* o, const void* gate, long long ld_g, const float* w, int T, int H, int Dv, float eps,
                                   int act, void* out, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long units = (long long)T * H;
    const int grid = (int)((units + 7) / 8);
    if (dtype == kF32) TTIE_LAUNCH(head_norm_gate_kernel<float>, grid, 256, 0, s, o, (const float*)gate, ld_g, w, T, H, Dv, eps, act, (float*)out);
    else if (dtype == kBF16) TTIE_LAUNCH(head_norm_gate_kernel<__nv_bfloat16>, grid, 256, 0, s, o, (const __nv_bfloat16*)gate, ld_g, w, T, H, Dv, eps, act, (__nv_bfloat16*)out);
    else TTIE_FAIL("head_norm_gate: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("head_norm_gate");
    return 0;
}
