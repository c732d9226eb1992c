// SwiGLU activation on the stacked gate|up product:  a[t, f] = silu(gu[t, f]) * gu[t, F + f],
// silu(g) = g * sigmoid(g), in 32-bit (src/transformer/ffn.zig:23-30, src/cuda/layer_kernels.cu:62-70).
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int F, size_t total) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F, f = i % F;
    const float g = to_float(gu[t * 2 * F + f]);
    const float u = to_float(gu[t * 2 * F + F + f]);
    out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// bfloat16 rows with F a multiple of 8: one thread per 8 outputs, 16-byte loads and stores
__global__ void silu_mul_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, int F8, size_t total8) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const size_t t = i / F8, f = (i % F8) * 8;
    const size_t F = (size_t)F8 * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + f);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + f);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(up[j]);
        // the fast exponential and division: their error (a few 2^-22) is far below the result's rounding to bfloat16
        op[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * F + f) = o4;
}

ZAI_API int zai_silu_mul(void* out, const void* gu, int dtype, int N, int F, cudaStream_t stream) {
    const size_t total = (size_t)N * F;
    if (total == 0) return ZAI_OK;
    const int threads = 256;
    if (dtype == ZAI_BF16 && (F & 7) == 0) {
        const size_t total8 = total / 8;
        return launch_pdl(silu_mul_bf16x8_kernel, dim3((unsigned)((total8 + threads - 1) / threads)), dim3(threads), 0,
                          stream, (bf16*)out, (const bf16*)gu, F / 8, total8);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    ZAI_DISPATCH(dtype, return launch_pdl(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (T*)out, (const T*)gu, F, total));
}

// ---- an activation on its own:  0 exact (erf) GELU, 1 tanh GELU, 2 SiLU, 3 ReLU; computed in 32-bit
__device__ __forceinline__ float zai_activate(float v, int kind) {
    switch (kind) {
        case 0: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        case 1: return 0.5f * v * (1.f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v)));
        case 2: return v / (1.f + expf(-v));
        default: return fmaxf(v, 0.f);
    }
}

// act(gate) * up on the stacked gate|up rows, for any of the activations above (SiLU has kernels of its own)
template <typename T>
__global__ void act_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int F, size_t total, int kind) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F, f = i % F;
    out[i] = from_float<T>(zai_activate(to_float(gu[t * 2 * F + f]), kind) * to_float(gu[t * 2 * F + F + f]));
}

ZAI_API int zai_act_mul(void* out, const void* gu, int dtype, int N, int F, int kind, cudaStream_t stream) {
    const size_t total = (size_t)N * F;
    if (total == 0) return ZAI_OK;
    if (kind < 0 || kind > 3) return ZAI_BAD_SIZE;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    ZAI_DISPATCH(dtype, return launch_pdl(act_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)gu, F, total, kind));
}

template <typename T>
__global__ void activation_kernel(T* __restrict__ out, const T* __restrict__ in, int kind, size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<T>(zai_activate(to_float(in[i]), kind));
}

__global__ void activation_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, int kind, size_t total8) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const uint4 v4 = *reinterpret_cast<const uint4*>(in + i * 8);
    const __nv_bfloat162* vp = reinterpret_cast<const __nv_bfloat162*>(&v4);
    uint4 o4;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(vp[j]);
        op[j] = __floats2bfloat162_rn(zai_activate(v.x, kind), zai_activate(v.y, kind));
    }
    *reinterpret_cast<uint4*>(out + i * 8) = o4;
}

ZAI_API int zai_activation(void* out, const void* in, int dtype, int kind, long long total, cudaStream_t stream) {
    if (total <= 0) return ZAI_OK;
    if (kind < 0 || kind > 3) return ZAI_BAD_SIZE;
    const int threads = 256;
    if (dtype == ZAI_BF16 && (total & 7) == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 15) == 0) {
        const size_t total8 = (size_t)total / 8;
        return launch_pdl(activation_bf16x8_kernel, dim3((unsigned)((total8 + threads - 1) / threads)), dim3(threads), 0, stream,
                          (bf16*)out, (const bf16*)in, kind, total8);
    }
    const unsigned blocks = (unsigned)(((size_t)total + threads - 1) / threads);
    ZAI_DISPATCH(dtype, return launch_pdl(activation_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (T*)out, (const T*)in, kind,
                                          (size_t)total));
}

// ---- out = wa * a + wb * b, in 32-bit, rounded once
template <typename T>
__global__ void weighted_sum_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, float wa, float wb,
                                    size_t total) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<T>(wa * to_float(a[i]) + wb * to_float(b[i]));
}

ZAI_API int zai_weighted_sum(void* out, const void* a, const void* b, int dtype, float wa, float wb, long long total,
                             cudaStream_t stream) {
    if (total <= 0) return ZAI_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)(((size_t)total + threads - 1) / threads);
    ZAI_DISPATCH(dtype, return launch_pdl(weighted_sum_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (T*)out, (const T*)a,
                                          (const T*)b, wa, wb, (size_t)total));
}

// ---- a gated activation with bounded branches on the stacked gate|up product, in 32-bit:
//   g = min(gu[t, f], limit);  u = clamp(gu[t, F + f], -limit, limit);  a[t, f] = g * sigmoid(alpha * g) * (u + 1)
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ gu, int F, size_t total, float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F, f = i % F;
    const float g = fminf(to_float(gu[t * 2 * F + f]), limit);
    const float u = fminf(fmaxf(to_float(gu[t * 2 * F + F + f]), -limit), limit);
    out[i] = from_float<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// bfloat16 rows with F a multiple of 8: one thread per 8 outputs, 16-byte loads and stores
__global__ void clamped_glu_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, int F8, size_t total8, float limit,
                                          float alpha) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const size_t t = i / F8, f = (i % F8) * 8;
    const size_t F = (size_t)F8 * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + f);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * F + F + f);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
    auto one = [&](float g, float u) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fdividef(g, 1.f + __expf(-alpha * g)) * (u + 1.f);
    };
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(up[j]);
        op[j] = __floats2bfloat162_rn(one(g.x, u.x), one(g.y, u.y));
    }
    *reinterpret_cast<uint4*>(out + t * F + f) = o4;
}

ZAI_API int zai_clamped_glu(void* out, const void* gu, int dtype, int N, int F, float limit, float alpha, cudaStream_t stream) {
    const size_t total = (size_t)N * F;
    if (total == 0) return ZAI_OK;
    const int threads = 256;
    if (dtype == ZAI_BF16 && (F & 7) == 0) {
        const size_t total8 = total / 8;
        return launch_pdl(clamped_glu_bf16x8_kernel, dim3((unsigned)((total8 + threads - 1) / threads)), dim3(threads), 0, stream,
                          (bf16*)out, (const bf16*)gu, F / 8, total8, limit, alpha);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    ZAI_DISPATCH(dtype, return launch_pdl(clamped_glu_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (T*)out, (const T*)gu, F, total,
                                          limit, alpha));
}

// ---- logits in place (32-bit):  x <- x * scale, then, with cap > 0,  x <- cap * tanh(x / cap)
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t total, float scale, float cap) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

ZAI_API int zai_scale_softcap(float* x, long long total, float scale, float cap, cudaStream_t stream) {
    if (total <= 0) return ZAI_OK;
    return launch_pdl(scale_softcap_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, (size_t)total, scale, cap);
}
