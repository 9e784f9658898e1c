// The recurrent block with a real-gated linear recurrent unit (RG-LRU), for any split of a sequence into steps.
// Per request the state row holds [taps, width] 32-bit values: row 0 is the recurrent state S, rows 1 .. taps-1 the last
// taps-1 inputs of the short convolution (oldest first).
//   causal_conv:  u[t, c] = sum_k w[c, k] * in[t - (taps-1) + k, c] + b[c]   (inputs before the step come from the state row,
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
            acc = fmaf(to_f32(cw[(size_t)c * taps + k]), v, acc);
        }
        u32[e] = acc;
        if (u_c) u_c[e] = from_f32<T>(acc);
    }
}

struct ScanArgs {
    const float* pre; const void* br; const void* bi; const void* lam; const float* u; const void* xin; long long ld_x; int col_x;
    const void* ypre; long long ld_y; int col_y; float* state; int state_rows; const int* qsl; const int* slot_ids;
    void* out; int T; int width; int taps; int bs; float decay_c; int num_seqs;
};

// (the pointers are passed as __restrict__ locals so that the loads of the next tokens may move above this token's store)
template <typename T, typename W>
__device__ __forceinline__ void gate_step(const ScanArgs& a, const float* __restrict__ pre, const float* __restrict__ u, int t, int c,
                                          int blk, int o, float br, float bi, float sp, float& av, float& bv) {
    const float* g = pre + ((size_t)blk * a.T + t) * (2 * a.bs);
    const float r = sigmoidf_(g[o] + br), i = sigmoidf_(g[a.bs + o] + bi);
    const float loga = -a.decay_c * r * sp;
    av = expf(loga);
    bv = sqrtf(-expm1f(2.0f * loga)) * i * u[(size_t)t * a.width + c];
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
#pragma unroll 4
    for (int t = q0; t < q0 + n; ++t) {
        float av, bv;
        gate_step<T, W>(a, pre, u, t, c, blk, o, br, bi, sp, av, bv);
        S = fmaf(av, S, bv);
        out[(size_t)t * a.width + c] = from_f32<T>(S * gelu_tanhf_(to_f32(ypre[(size_t)t * a.ld_y + a.col_y + c])));
    }
    row[c] = S;
    move_tail<T>(a, row, q0, n, c);
}

// ---- the chunked form.  Pass 1: per (chunk, channel) the recurrence over the chunk from S = 0: A = prod a, B = the state it
// would reach.  Pass 2: per (request, channel) carry S over the chunk edges (S_edge <- A * S_edge + B), keeping the state at
// every chunk's start.  Pass 3: per (chunk, channel) the recurrence again from the chunk's start state, writing the outputs.
constexpr int CHUNK = 32;

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
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float av, bv;
        gate_step<T, W>(a, pre, u, t, c, blk, o, br, bi, sp, av, bv);
        A *= av;
        B = fmaf(av, B, bv);
    }
    ab[(size_t)k * a.width + c] = make_float2(A, B);
}

template <typename T>
__global__ void __launch_bounds__(128)
rglru_chunk_carry_kernel(ScanArgs a, const int* __restrict__ seq_chunk0, float2* __restrict__ ab) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= a.width) return;
    const int q0 = a.qsl[s], n = a.qsl[s + 1] - q0;
    if (n <= 0) return;
    float* row = a.state + (size_t)slot_row(a.slot_ids[s], a.state_rows) * a.taps * a.width;
    float S = row[c];
    const int k0 = seq_chunk0[s], nk = (n + CHUNK - 1) / CHUNK;
    int k = k0;
    for (; k + 4 <= k0 + nk; k += 4) {                               // four chunks' pairs in flight: the chain is the fma, not the loads
        float2 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = ab[(size_t)(k + j) * a.width + c];
#pragma unroll
        for (int j = 0; j < 4; ++j) { ab[(size_t)(k + j) * a.width + c].x = S; S = fmaf(v[j].x, S, v[j].y); }
    }
    for (; k < k0 + nk; ++k) {
        const float2 v = ab[(size_t)k * a.width + c];
        ab[(size_t)k * a.width + c].x = S;                           // the state this chunk starts from
        S = fmaf(v.x, S, v.y);
    }
    row[c] = S;
    move_tail<T>(a, row, q0, n, c);
}

template <typename T, typename W>
__global__ void __launch_bounds__(128)
rglru_chunk_apply_kernel(ScanArgs a, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_t0, const float2* __restrict__ ab) {
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
    float S = ab[(size_t)k * a.width + c].x;
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float av, bv;
        gate_step<T, W>(a, pre, u, t, c, blk, o, br, bi, sp, av, bv);
        S = fmaf(av, S, bv);
        out[(size_t)t * a.width + c] = from_f32<T>(S * gelu_tanhf_(to_f32(ypre[(size_t)t * a.ld_y + a.col_y + c])));
    }
}

// chunk table of a step, built on the device from query_start_loc: chunk k belongs to request chunk_seq[k] (-1: unused) and
// starts at token chunk_t0[k]; request s owns chunks seq_chunk0[s] ... (one thread: a step has few requests)
__global__ void rglru_chunk_table_kernel(const int* __restrict__ qsl, int num_seqs, int max_chunks, int* __restrict__ chunk_seq,
                                         int* __restrict__ chunk_t0, int* __restrict__ seq_chunk0) {
    TTIE_PDL_ENTRY();
    if (threadIdx.x || blockIdx.x) return;
    int k = 0;
    for (int s = 0; s < num_seqs; ++s) {
        seq_chunk0[s] = k;
        for (int t = qsl[s]; t < qsl[s + 1] && k < max_chunks; t += CHUNK, ++k) { chunk_seq[k] = s; chunk_t0[k] = t; }
    }
    for (; k < max_chunks; ++k) { chunk_seq[k] = -1; chunk_t0[k] = 0; }
}

inline int grid_for(size_t total) { return (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192); }
}  // namespace

extern "C" int ttie_causal_conv(const void* in, long long ld, int col0, int T, int width, int taps, const void* cw, const void* cb,
                                int w_dtype, const float* state, int state_rows, const int* token_seq, const int* qsl,
                                const int* slot_ids, float* u32, void* u_c, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (taps < 1) TTIE_FAIL("causal_conv: %d taps", taps);
    cudaStream_t s = (cudaStream_t)stream;
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
// num_seqs words followed (8-byte aligned) by float2 [max_chunks, width], with max_chunks >= sum over requests of ceil(n / chunk).
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
    TTIE_LAUNCH(rglru_chunk_table_kernel, 1, 32, 0, s, qsl, num_seqs, max_chunks, chunk_seq, chunk_t0, seq_chunk0);
    const dim3 grid_chunk(ceil_div(width, 128), max_chunks);
#define RD(TT, WW) TTIE_LAUNCH((rglru_chunk_reduce_kernel<TT, WW>), grid_chunk, 128, 0, s, a, chunk_seq, chunk_t0, ab)
    if (dtype == kF32) RD(float, float); else if (vec_dtype == kF32) RD(__nv_bfloat16, float); else RD(__nv_bfloat16, __nv_bfloat16);
#undef RD
    if (dtype == kF32) TTIE_LAUNCH(rglru_chunk_carry_kernel<float>, grid_seq, 128, 0, s, a, seq_chunk0, ab);
    else TTIE_LAUNCH(rglru_chunk_carry_kernel<__nv_bfloat16>, grid_seq, 128, 0, s, a, seq_chunk0, ab);
#define AP(TT, WW) TTIE_LAUNCH((rglru_chunk_apply_kernel<TT, WW>), grid_chunk, 128, 0, s, a, chunk_seq, chunk_t0, ab)
    if (dtype == kF32) AP(float, float); else if (vec_dtype == kF32) AP(__nv_bfloat16, float); else AP(__nv_bfloat16, __nv_bfloat16);
#undef AP
    TTIE_CHECK_LAUNCH("rglru_scan (chunked)");
    return 0;
}
