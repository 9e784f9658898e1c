// The recurrent block with a real-gated linear recurrent unit (RG-LRU), for any split of a sequence into steps.
// Per request the state row holds [taps, width] 32-bit values: row 0 is the recurrent state S, rows 1 .. taps-1 the last
// taps-1 inputs of the short convolution (oldest first).
//   causal_conv:  u[t, c] = sum_k w[k, c] * in[t - (taps-1) + k, c] + b[c]   (weights tap-major; inputs before the step come from the state row,
//                 zeros before the sequence's start because a fresh row is zero); one thread per (token, channel)
//   rglru_scan:   r = sigmoid(pre_r + br), i = sigmoid(pre_i + bi), log a = -c * r * softplus(lam), a = exp(log a),
//                 S <- a * S + sqrt(1 - a^2) * i * u,  out = S * gelu_tanh(y_pre); all 32-bit; it also moves the convolution's
//                 inputs of this step into the state row.  Two forms: one thread per (request, channel) walking the tokens
//                 (steps of few tokens), and a chunked form for long portions: every chunk of tokens reduces its recurrence
//                 to (product of a, accumulated input) in parallel, a second pass carries S over the chunk edges.
// Gate pre-activations come as [blocks, T, 2 * bs] (the block-diagonal products, r first then i within a block).
#include "common.cuh"
using namespace ttie;

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ int slot_row(int slot, int num_rows) { return slot < 0 ? num_rows - 1 : slot; }

template <typename T, typename W>
__global__ void causal_conv_kernel(const T* __restrict__ in, long long ld, int col0, int T_, int width, int taps,
                                   const W* __restrict__ cw, const W* __restrict__ cb, const float* __restrict__ state,
                                   int state_rows, const int* __restrict__ token_seq, const int* __restrict__ qsl,
                                   const int* __restrict__ slot_ids, float* __restrict__ u32, T* __restrict__ u_c) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;             // grid: (channels, tokens)
    if (c >= width) return;
    for (int t = blockIdx.y; t < T_; t += gridDim.y) {
        const size_t e = (size_t)t * width + c;
        const int s = token_seq[t];
        const int j = t - qsl[s];                                   // index within the request's tokens of this step
        const float* tail = state + ((size_t)slot_row(slot_ids[s], state_rows) * taps + 1) * width;
        float acc = cb ? to_f32(cb[c]) : 0.f;
        for (int k = 0; k < taps; ++k) {
            const int src = j - (taps - 1) + k;
            const float v = src >= 0 ? to_f32(in[(size_t)(t - j + src) * ld + col0 + c]) : tail[(size_t)(taps - 1 + src) * width + c];
            acc = fmaf(to_f32(cw[(size_t)k * width + c]), v, acc);
        }
        u32[e] = acc;
        if (u_c) u_c[e] = from_f32<T>(acc);
    }
}

__device__ __forceinline__ void load8(const float* p, float* o) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* o) {
    const uint4 x = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}

// bfloat16 inputs, eight channels per thread (width, the input's row stride and first column multiples of 8)
template <typename W>
__global__ void __launch_bounds__(128)
causal_conv_vec8_kernel(const __nv_bfloat16* __restrict__ in, long long ld, int col0, int T_, int width, int taps,
                        const W* __restrict__ cw, const W* __restrict__ cb, const float* __restrict__ state, int state_rows,
                        const int* __restrict__ token_seq, const int* __restrict__ qsl, const int* __restrict__ slot_ids,
                        float* __restrict__ u32, __nv_bfloat16* __restrict__ u_c) {
    TTIE_PDL_ENTRY();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= width) return;
    for (int t = blockIdx.y; t < T_; t += gridDim.y) {
        const int s = token_seq[t];
        const int j = t - qsl[s];
        const float* tail = state + ((size_t)slot_row(slot_ids[s], state_rows) * taps + 1) * width;
        float acc[8];
        if (cb) load8(cb + c, acc);
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        }
        for (int k = 0; k < taps; ++k) {
            const int src = j - (taps - 1) + k;
            float v[8];
            if (src >= 0) {
                const uint4 x = *reinterpret_cast<const uint4*>(in + (size_t)(t - j + src) * ld + col0 + c);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
            } else {
                const float4 a = *reinterpret_cast<const float4*>(tail + (size_t)(taps - 1 + src) * width + c);
                const float4 b = *reinterpret_cast<const float4*>(tail + (size_t)(taps - 1 + src) * width + c + 4);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
            float w[8];
            load8(cw + (size_t)k * width + c, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[i], v[i], acc[i]);
        }
        float* o = u32 + (size_t)t * width + c;
        *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
        if (u_c) {
            uint4 p;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&p);
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            *reinterpret_cast<uint4*>(u_c + (size_t)t * width + c) = p;
        }
    }
}

struct ScanArgs {
    const float* pre; const void* br; const void* bi; const void* lam; const float* u; const void* xin; long long ld_x; int col_x;
    const void* ypre; long long ld_y; int col_y; float* state; int state_rows; const int* qsl; const int* slot_ids;
    void* out; int T; int width; int taps; int bs; float decay_c; int num_seqs;
};

// The tokens of a thread's range are taken GROUP at a time: first every load of the group is issued (gate pre-activations,
// convolution output, the other branch), then the group's recurrence runs from registers - the chain is then arithmetic only,
// and a thread keeps 4 * GROUP loads in flight (these kernels have few warps per SM; what they wait for is memory).
constexpr int GROUP = 8;
struct Gates { float r[GROUP], i[GROUP], u[GROUP]; };

__device__ __forceinline__ void load_gates(const ScanArgs& a, const float* __restrict__ pre, const float* __restrict__ u, int t, int t_end,
                                           int c, int blk, int o, Gates& g) {
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
        const int tt = min(t + j, t_end - 1);
        const float* p = pre + ((size_t)blk * a.T + tt) * (2 * a.bs);
        g.r[j] = p[o]; g.i[j] = p[a.bs + o]; g.u[j] = u[(size_t)tt * a.width + c];
    }
}

// The arithmetic of a token.  A 32-bit run uses the library's accurate functions (and 1 - a^2 as -expm1(2 log a), which keeps
// its digits when a is close to 1).  A bfloat16 run computes the same 32-bit formulas with the hardware's exponential and
// reciprocal (relative error about 1e-6, far below the rounding of the bfloat16 operands around them): these kernels are bound
// by instruction issue, and the accurate functions cost four times as many instructions.
template <typename T> struct Arith {
    static __device__ __forceinline__ float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
    static __device__ __forceinline__ float exp_(float x) { return expf(x); }
    static __device__ __forceinline__ float one_minus_sq(float loga, float a) { return -expm1f(2.0f * loga); }
    static __device__ __forceinline__ float gelu(float z) { return gelu_tanhf_(z); }
};
template <> struct Arith<__nv_bfloat16> {
    static __device__ __forceinline__ float sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
    static __device__ __forceinline__ float exp_(float x) { return __expf(x); }
    static __device__ __forceinline__ float one_minus_sq(float loga, float a) { return fmaf(-a, a, 1.0f); }
    // 0.5 z (1 + tanh(k)) = z * sigmoid(2 k)
    static __device__ __forceinline__ float gelu(float z) { return z * sigmoid(1.5957691216057308f * (z + 0.044715f * z * z * z)); }
};

template <typename T>
__device__ __forceinline__ void gate_step(const ScanArgs& a, const Gates& g, int j, float br, float bi, float sp, float& av, float& bv) {
    const float r = Arith<T>::sigmoid(g.r[j] + br), i = Arith<T>::sigmoid(g.i[j] + bi);
    const float loga = -a.decay_c * r * sp;
    av = Arith<T>::exp_(loga);
    bv = sqrtf(Arith<T>::one_minus_sq(loga, av)) * i * g.u[j];
}

template <typename T>
__device__ __forceinline__ void move_tail(const ScanArgs& a, float* row, int q0, int n, int c) {
    // the convolution's last taps-1 inputs, oldest first: those of this step, and before them what the row held
    float* tail = row + a.width;
    const T* xin = (const T*)a.xin;
    for (int j = 0; j < a.taps - 1; ++j) {
        const int src = n - (a.taps - 1) + j;
        tail[(size_t)j * a.width + c] = src >= 0 ? to_f32(xin[(size_t)(q0 + src) * a.ld_x + a.col_x + c]) : tail[(size_t)(j + n) * a.width + c];
    }
}

// one thread per (request, channel), tokens in order
template <typename T, typename W>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(ScanArgs a) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= a.width) return;
    const int q0 = a.qsl[s], n = a.qsl[s + 1] - q0;
    if (n <= 0) return;
    float* row = a.state + (size_t)slot_row(a.slot_ids[s], a.state_rows) * a.taps * a.width;
    const int blk = c / a.bs, o = c % a.bs;
    const float* __restrict__ pre = a.pre;
    const float* __restrict__ u = a.u;
    const float br = to_f32(((const W*)a.br)[c]), bi = to_f32(((const W*)a.bi)[c]), sp = softplusf_(to_f32(((const W*)a.lam)[c]));
    const T* __restrict__ ypre = (const T*)a.ypre;
    T* __restrict__ out = (T*)a.out;
    float S = row[c];
    for (int t = q0; t < q0 + n; t += GROUP) {
        Gates g;
        float y[GROUP];
        load_gates(a, pre, u, t, q0 + n, c, blk, o, g);
#pragma unroll
        for (int j = 0; j < GROUP; ++j) y[j] = to_f32(ypre[(size_t)min(t + j, q0 + n - 1) * a.ld_y + a.col_y + c]);
#pragma unroll
        for (int j = 0; j < GROUP; ++j) {
            if (t + j >= q0 + n) break;
            float av, bv;
            gate_step<T>(a, g, j, br, bi, sp, av, bv);
            S = fmaf(av, S, bv);
            out[(size_t)(t + j) * a.width + c] = from_f32<T>(S * Arith<T>::gelu(y[j]));
        }
    }
    row[c] = S;
    move_tail<T>(a, row, q0, n, c);
}

// ---- the chunked form.  Pass 1: per (chunk, channel) the recurrence over the chunk from S = 0: A = prod a, B = the state it
// would reach.  Pass 2: per (request, channel) carry S over the chunk edges (S_edge <- A * S_edge + B), keeping the state at
// every chunk's start.  Pass 3: per (chunk, channel) the recurrence again from the chunk's start state, writing the outputs.
constexpr int CHUNK = 16;

template <typename T, typename W>
__global__ void __launch_bounds__(128)
rglru_chunk_reduce_kernel(ScanArgs a, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_t0, float2* __restrict__ ab) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= a.width) return;
    const int s = chunk_seq[k];
    if (s < 0) return;
    const int t0 = chunk_t0[k], t1 = min(t0 + CHUNK, a.qsl[s + 1]);
    const int blk = c / a.bs, o = c % a.bs;
    const float* __restrict__ pre = a.pre;
    const float* __restrict__ u = a.u;
    const float br = to_f32(((const W*)a.br)[c]), bi = to_f32(((const W*)a.bi)[c]), sp = softplusf_(to_f32(((const W*)a.lam)[c]));
    float A = 1.f, B = 0.f;
    for (int t = t0; t < t1; t += GROUP) {
        Gates g;
        load_gates(a, pre, u, t, t1, c, blk, o, g);
#pragma unroll
        for (int j = 0; j < GROUP; ++j) {
            if (t + j >= t1) break;
            float av, bv;
            gate_step<T>(a, g, j, br, bi, sp, av, bv);
            A *= av;
            B = fmaf(av, B, bv);
        }
    }
    ab[(size_t)k * a.width + c] = make_float2(A, B);
}

// The chain over a request's chunks is short work for few threads (one per request and channel), so it is cut once more: a
// CTA takes CC channels, its CG thread groups each compose their share of the chunks' pairs - (A, B) after (A', B') is
// (A A', A B' + B) - with the loads ahead of the arithmetic; one group then walks the CG totals in shared memory, and every
// group replays its share from its start state, writing the state each chunk starts from.
constexpr int CG = 16, CC = 16;
template <typename T>
__global__ void __launch_bounds__(CG * CC)
rglru_chunk_carry_kernel(ScanArgs a, const int* __restrict__ seq_chunk0, const float2* __restrict__ ab, float* __restrict__ start) {
    __shared__ float2 total[CG][CC];
    __shared__ float first[CG][CC];
    TTIE_PDL_ENTRY();
    const int cl = threadIdx.x % CC, g = threadIdx.x / CC, c = blockIdx.x * CC + cl, s = blockIdx.y;
    const int q0 = a.qsl[s], n = a.qsl[s + 1] - q0;
    if (n <= 0) return;                                              // (the same for the whole CTA)
    const bool valid = c < a.width;
    const int k0 = seq_chunk0[s], K = (n + CHUNK - 1) / CHUNK, per = (K + CG - 1) / CG;
    const int ka = k0 + g * per, kb = min(ka + per, k0 + K);
    constexpr int AHEAD = 8;
    float A = 1.f, B = 0.f;
    if (valid)
        for (int k = ka; k < kb; k += AHEAD) {
            float2 v[AHEAD];
#pragma unroll
            for (int j = 0; j < AHEAD; ++j) v[j] = ab[(size_t)min(k + j, kb - 1) * a.width + c];
#pragma unroll
            for (int j = 0; j < AHEAD; ++j)
                if (k + j < kb) { A *= v[j].x; B = fmaf(v[j].x, B, v[j].y); }
        }
    total[g][cl] = make_float2(A, B);
    __syncthreads();
    if (g == 0 && valid) {
        float* row = a.state + (size_t)slot_row(a.slot_ids[s], a.state_rows) * a.taps * a.width;
        float S = row[c];
        for (int gg = 0; gg < CG; ++gg) { first[gg][cl] = S; S = fmaf(total[gg][cl].x, S, total[gg][cl].y); }
        row[c] = S;
        move_tail<T>(a, row, q0, n, c);
    }
    __syncthreads();
    if (!valid) return;
    float S = first[g][cl];
    for (int k = ka; k < kb; k += AHEAD) {
        float2 v[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) v[j] = ab[(size_t)min(k + j, kb - 1) * a.width + c];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j)
            if (k + j < kb) { start[(size_t)(k + j) * a.width + c] = S; S = fmaf(v[j].x, S, v[j].y); }
    }
}

template <typename T, typename W>
__global__ void __launch_bounds__(128)
rglru_chunk_apply_kernel(ScanArgs a, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_t0, const float* __restrict__ start) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= a.width) return;
    const int s = chunk_seq[k];
    if (s < 0) return;
    const int t0 = chunk_t0[k], t1 = min(t0 + CHUNK, a.qsl[s + 1]);
    const int blk = c / a.bs, o = c % a.bs;
    const float* __restrict__ pre = a.pre;
    const float* __restrict__ u = a.u;
    const float br = to_f32(((const W*)a.br)[c]), bi = to_f32(((const W*)a.bi)[c]), sp = softplusf_(to_f32(((const W*)a.lam)[c]));
    const T* __restrict__ ypre = (const T*)a.ypre;
    T* __restrict__ out = (T*)a.out;
    float S = start[(size_t)k * a.width + c];
    for (int t = t0; t < t1; t += GROUP) {
        Gates g;
        float y[GROUP];
        load_gates(a, pre, u, t, t1, c, blk, o, g);
#pragma unroll
        for (int j = 0; j < GROUP; ++j) y[j] = to_f32(ypre[(size_t)min(t + j, t1 - 1) * a.ld_y + a.col_y + c]);
#pragma unroll
        for (int j = 0; j < GROUP; ++j) {
            if (t + j >= t1) break;
            float av, bv;
            gate_step<T>(a, g, j, br, bi, sp, av, bv);
            S = fmaf(av, S, bv);
            out[(size_t)(t + j) * a.width + c] = from_f32<T>(S * Arith<T>::gelu(y[j]));
        }
    }
}

// chunk table of a step, built on the device from query_start_loc: chunk k belongs to request chunk_seq[k] (-1: unused) and
// starts at token chunk_t0[k]; request s owns chunks seq_chunk0[s] ...  One thread per chunk (and per request) adds up the
// requests' chunk counts before its own: a step has few requests.
__global__ void rglru_chunk_table_kernel(const int* __restrict__ qsl, int num_seqs, int max_chunks, int* __restrict__ chunk_seq,
                                         int* __restrict__ chunk_t0, int* __restrict__ seq_chunk0) {
    TTIE_PDL_ENTRY();
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k < num_seqs) {
        int at = 0;
        for (int s = 0; s < k; ++s) at += (qsl[s + 1] - qsl[s] + CHUNK - 1) / CHUNK;
        seq_chunk0[k] = at;
    }
    if (k >= max_chunks) return;
    int at = 0, owner = -1, t0 = 0;
    for (int s = 0; s < num_seqs; ++s) {
        const int nk = (qsl[s + 1] - qsl[s] + CHUNK - 1) / CHUNK;
        if (k < at + nk) { owner = s; t0 = qsl[s] + (k - at) * CHUNK; break; }
        at += nk;
    }
    chunk_seq[k] = owner; chunk_t0[k] = t0;
}

inline int grid_for(size_t total) { return (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192); }
}  // namespace

extern "C" int ttie_causal_conv(const void* in, long long ld, int col0, int T, int width, int taps, const void* cw, const void* cb,
                                int w_dtype, const float* state, int state_rows, const int* token_seq, const int* qsl,
                                const int* slot_ids, float* u32, void* u_c, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (taps < 1) TTIE_FAIL("causal_conv: %d taps", taps);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kBF16 && width % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 && ((((uintptr_t)in) | ((uintptr_t)state) | ((uintptr_t)u32) | ((uintptr_t)u_c) | ((uintptr_t)cw) | ((uintptr_t)cb)) & 15) == 0) {
        const dim3 g8(ceil_div(width / 8, 128), T < 65535 ? T : 65535);
        if (w_dtype == kF32) TTIE_LAUNCH(causal_conv_vec8_kernel<float>, g8, 128, 0, s, (const __nv_bfloat16*)in, ld, col0, T, width, taps, (const float*)cw,
                                         (const float*)cb, state, state_rows, token_seq, qsl, slot_ids, u32, (__nv_bfloat16*)u_c);
        else TTIE_LAUNCH(causal_conv_vec8_kernel<__nv_bfloat16>, g8, 128, 0, s, (const __nv_bfloat16*)in, ld, col0, T, width, taps, (const __nv_bfloat16*)cw,
                         (const __nv_bfloat16*)cb, state, state_rows, token_seq, qsl, slot_ids, u32, (__nv_bfloat16*)u_c);
        TTIE_CHECK_LAUNCH("causal_conv");
        return 0;
    }
    const dim3 grid(ceil_div(width, 256), T < 65535 ? T : 65535);
#define CC(TT, WW) TTIE_LAUNCH((causal_conv_kernel<TT, WW>), grid, 256, 0, s, (const TT*)in, ld, col0, T, width, taps, (const WW*)cw, \
                               (const WW*)cb, state, state_rows, token_seq, qsl, slot_ids, u32, (TT*)u_c)
    if (dtype == kF32) { if (w_dtype != kF32) TTIE_FAIL("causal_conv: a 32-bit run needs 32-bit weights"); CC(float, float); }
    else if (w_dtype == kF32) CC(__nv_bfloat16, float);
    else CC(__nv_bfloat16, __nv_bfloat16);
#undef CC
    TTIE_CHECK_LAUNCH("causal_conv");
    return 0;
}

extern "C" int ttie_rglru_chunk() { return CHUNK; }

// vec_dtype: dtype of br, bi and lam.  chunk_ws: null for the token-by-token form; else int32 scratch of 2 * max_chunks +
// num_seqs words and float [max_chunks, width, 3] (the chunks' pairs, then their start states), with max_chunks >= sum over requests of ceil(n / chunk).
extern "C" int ttie_rglru_scan(const float* pre, const void* br, const void* bi, const void* lam, int vec_dtype, const float* u,
                               const void* xin, long long ld_x, int col_x, const void* ypre, long long ld_y, int col_y,
                               float* state, int state_rows, const int* qsl, const int* slot_ids, int num_seqs, void* out, int T,
                               int width, int taps, int bs, float decay_c, int* chunk_ws, int max_chunks, void* ab_ws,
                               int dtype, void* stream) {
    if (T <= 0 || num_seqs <= 0) return 0;
    if (bs <= 0 || width % bs) TTIE_FAIL("rglru_scan: width %d is not a multiple of the block size %d", width, bs);
    cudaStream_t s = (cudaStream_t)stream;
    ScanArgs a{pre, br, bi, lam, u, xin, ld_x, col_x, ypre, ld_y, col_y, state, state_rows, qsl, slot_ids, out, T, width, taps, bs, decay_c, num_seqs};
    const dim3 grid_seq(ceil_div(width, 128), num_seqs);
    if (dtype == kF32 && vec_dtype != kF32) TTIE_FAIL("rglru_scan: a 32-bit run needs 32-bit vectors");
    if (!chunk_ws) {
#define SC(TT, WW) TTIE_LAUNCH((rglru_scan_kernel<TT, WW>), grid_seq, 128, 0, s, a)
        if (dtype == kF32) SC(float, float); else if (vec_dtype == kF32) SC(__nv_bfloat16, float); else SC(__nv_bfloat16, __nv_bfloat16);
#undef SC
        TTIE_CHECK_LAUNCH("rglru_scan");
        return 0;
    }
    int* chunk_seq = chunk_ws; int* chunk_t0 = chunk_ws + max_chunks; int* seq_chunk0 = chunk_ws + 2 * max_chunks;
    float2* ab = (float2*)ab_ws;
    float* start = (float*)(ab + (size_t)max_chunks * width);
    TTIE_LAUNCH(rglru_chunk_table_kernel, ceil_div(max_chunks > num_seqs ? max_chunks : num_seqs, 128), 128, 0, s, qsl, num_seqs, max_chunks, chunk_seq, chunk_t0, seq_chunk0);
    const dim3 grid_chunk(ceil_div(width, 128), max_chunks);
#define RD(TT, WW) TTIE_LAUNCH((rglru_chunk_reduce_kernel<TT, WW>), grid_chunk, 128, 0, s, a, chunk_seq, chunk_t0, ab)
    if (dtype == kF32) RD(float, float); else if (vec_dtype == kF32) RD(__nv_bfloat16, float); else RD(__nv_bfloat16, __nv_bfloat16);
#undef RD
    const dim3 grid_carry(ceil_div(width, CC), num_seqs);
    if (dtype == kF32) TTIE_LAUNCH(rglru_chunk_carry_kernel<float>, grid_carry, CG * CC, 0, s, a, seq_chunk0, ab, start);
    else TTIE_LAUNCH(rglru_chunk_carry_kernel<__nv_bfloat16>, grid_carry, CG * CC, 0, s, a, seq_chunk0, ab, start);
#define AP(TT, WW) TTIE_LAUNCH((rglru_chunk_apply_kernel<TT, WW>), grid_chunk, 128, 0, s, a, chunk_seq, chunk_t0, start)
    if (dtype == kF32) AP(float, float); else if (vec_dtype == kF32) AP(__nv_bfloat16, float); else AP(__nv_bfloat16, __nv_bfloat16);
#undef AP
    TTIE_CHECK_LAUNCH("rglru_scan (chunked)");
    return 0;
}
