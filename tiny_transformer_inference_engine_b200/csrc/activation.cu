// Elementwise functions between products, evaluated in 32-bit: out[i] = f(in[i]) for contiguous arrays, input and output
// each float32 or bfloat16 (in place when they are the same array).
//   0  relu(x)^2          1  tanh(x)          2  c * tanh(x / c)   (a soft cap at +-c)
#include "common.cuh"
#include <math.h>
using namespace ttie;

namespace {

__device__ __forceinline__ float apply(float x, int kind, float c) {
    if (kind == 0) { const float r = fmaxf(x, 0.f); return r * r; }
    if (kind == 1) return tanhf(x);
    return c * tanhf(x / c);
}

template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n, int kind, float c) {
    TTIE_PDL_ENTRY();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(apply(to_f32(in[i]), kind, c));
}

// bfloat16 to bfloat16, eight values per thread (n a multiple of 8, both arrays 16-byte aligned)
__global__ void activation_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long n8, int kind, float c) {
    TTIE_PDL_ENTRY();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const uint4 x = in[i];
        uint4 y;
        const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&x);
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(a[k]);
            b[k] = __floats2bfloat162_rn(apply(f.x, kind, c), apply(f.y, kind, c));
        }
        out[i] = y;
    }
}

}  // namespace

extern "C" int ttie_activation(const void* in, void* out, long long n, int kind, float c, int in_dtype, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 2) TTIE_FAIL("activation: unknown kind %d", kind);
    if (kind == 2 && !(c > 0.f)) TTIE_FAIL("activation: a soft cap needs a positive constant");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    if (in_dtype == kBF16 && out_dtype == kBF16 && n % 8 == 0 && !(((uintptr_t)in | (uintptr_t)out) & 15)) {
        const long long n8 = n / 8;
        const int grid = (int)((n8 + threads - 1) / threads < 148LL * 16 ? (n8 + threads - 1) / threads : 148LL * 16);
        TTIE_LAUNCH(activation_bf16x8_kernel, grid, threads, 0, s, (const uint4*)in, (uint4*)out, n8, kind, c);
        TTIE_CHECK_LAUNCH("activation");
        return 0;
    }
    const int grid = (int)((n + threads - 1) / threads < 148LL * 32 ? (n + threads - 1) / threads : 148LL * 32);
    if (in_dtype == kF32 && out_dtype == kF32) TTIE_LAUNCH((activation_kernel<float, float>), grid, threads, 0, s, (const float*)in, (float*)out, n, kind, c);
    else if (in_dtype == kF32 && out_dtype == kBF16) TTIE_LAUNCH((activation_kernel<float, __nv_bfloat16>), grid, threads, 0, s, (const float*)in, (__nv_bfloat16*)out, n, kind, c);
    else if (in_dtype == kBF16 && out_dtype == kBF16) TTIE_LAUNCH((activation_kernel<__nv_bfloat16, __nv_bfloat16>), grid, threads, 0, s, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, n, kind, c);
    else if (in_dtype == kBF16 && out_dtype == kF32) TTIE_LAUNCH((activation_kernel<__nv_bfloat16, float>), grid, threads, 0, s, (const __nv_bfloat16*)in, (float*)out, n, kind, c);
    else TTIE_FAIL("activation: unknown dtypes %d -> %d", in_dtype, out_dtype);
    TTIE_CHECK_LAUNCH("activation");
    return 0;
}
