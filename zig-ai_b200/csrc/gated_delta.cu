// Gated delta rule: per head a state matrix S [D, V] in 32-bit, carried between steps.  For each token
//
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// (the read-out sees the token's own write), with q and k unit vectors per head (q also times D^-1/2),
// beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)): one decay per head, or (`channel`) one per head and
// key channel, g [H, D], which then scales the rows of S one by one (a and dt_bias are [H D] wide, A_log stays per
// head).  The output gate is silu or (`gate_act` 1) a sigmoid.  A step of single tokens is one kernel (a block per
// request and head does all of it); steps with portions run three kernels:
//   * prepare: unit norms, beta and g for every row of the step, all 32-bit;
//   * the recurrence: the columns of S are independent, so a block owns some columns of one head of one
//     request and walks the request's rows in order; P lanes of a warp share a column, each with DP of
//     its D rows in registers; the operands of the next sixteen tokens come into shared memory by
//     asynchronous copies while the current sixteen are computed;
//   * the output norm: o / rms(o) * weight * silu(gate) per head, rounded to the model's dtype.
#include <cstdlib>
#include "common.cuh"

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// qk_out [N, 2, G, D]: q then k, unit length (+ eps inside the root), q times D^-1/2;  bg_out [N, 2, H]: beta, g
// gch_out (channel decays only) [N, H, D]: g per head and key channel; bg_out then holds beta alone
template <typename T>
__global__ void delta_prepare_kernel(float* __restrict__ qk_out, float* __restrict__ bg_out, float* __restrict__ gch_out,
                                     const T* __restrict__ qkv, int qkv_stride, const T* __restrict__ b_in, int b_stride,
                                     const T* __restrict__ a_in, int a_stride, const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias, int H, int G, int D, float unit_eps) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const float q_scale = rsqrtf((float)D);
    for (int item = warp; item < 2 * G; item += nwarp) {
        const T* src = qkv + (size_t)t * qkv_stride + (size_t)item * D;       // q heads, then k heads
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float v = to_float(src[d]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss + unit_eps) * (item < G ? q_scale : 1.f);
        float* dst = qk_out + ((size_t)t * 2 * G + item) * D;
        for (int d = lane; d < D; d += 32) dst[d] = to_float(src[d]) * inv;
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const float b = to_float(b_in[(size_t)t * b_stride + h]);
        bg_out[(size_t)t * 2 * H + h] = 1.f / (1.f + expf(-b));
        if (!gch_out) {
            const float a = to_float(a_in[(size_t)t * a_stride + h]);
            bg_out[(size_t)t * 2 * H + H + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
        }
    }
    if (gch_out) {
        for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
            const float a = to_float(a_in[(size_t)t * a_stride + i]);
            gch_out[(size_t)t * H * D + i] = expf(-expf(a_log[i / D]) * softplus_f(a + dt_bias[i]));
        }
    }
}

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// The operands of TB tokens (a stage of the ring; fewer where a head is large, so that two stages fit) in shared memory: per token k and q of the head (each P groups of DP values,
// a group padded to DP + 4 so that the P groups read by one warp lie in different banks, 16-byte aligned), beta, g,
// and the block's columns of v as 32-bit values.
// With channel decays a token also brings its head's D decays (a third group laid out like k and q), and a stage holds
// fewer tokens where a head is large.
template <int DP, int P, bool CH>
struct DeltaStage {
    static constexpr int GROUP = DP + 4, KQ = P * GROUP, VB = 128 / P, NG = CH ? 3 : 2, PER_TOKEN = NG * KQ + 4 + VB;
    static constexpr int TB = CH ? (DP * P > 128 ? 4 : (DP * P > 64 ? 8 : 16)) : (DP * P > 128 ? 8 : 16);
};

template <typename T, int DP, int P, bool CH>
__global__ void __launch_bounds__(128) gated_delta_kernel(
    float* __restrict__ o_out, const float* __restrict__ qk, const float* __restrict__ bg, const float* __restrict__ gch,
    const T* __restrict__ v_in,
    int v_stride, float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ slot_ids, int H, int G,
    int D, int V, int write_state, int num_slots, int* __restrict__ status) {
    using St = DeltaStage<DP, P, CH>;
    constexpr int VB = St::VB, TB = St::TB, NG = St::NG;
    __shared__ __align__(16) float ring[2][TB][St::PER_TOKEN];
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, p = threadIdx.x % P, jl = threadIdx.x / P;
    const int j0 = blockIdx.z * VB;
    int j = j0 + jl;
    const bool live = j < V;
    if (!live) j = V - 1;                              // (stays for the shuffles, stores nothing)
    const int start = cu_q[seq], end = cu_q[seq + 1];
    if (end <= start) return;
    const int slot = zai_checked_slot(slot_ids[seq], num_slots, status);
    const int kvh = h / (H / G), d0 = p * DP;
    float* st = state + (((size_t)slot * H + h) * D) * V + j;
    float S[DP];
#pragma unroll
    for (int i = 0; i < DP; ++i) S[i] = d0 + i < D ? st[(size_t)(d0 + i) * V] : 0.f;
    for (int i = threadIdx.x; i < 2 * TB * St::PER_TOKEN; i += 128) (&ring[0][0][0])[i] = 0.f;   // rows of k, q beyond D stay zero
    __syncthreads();

    // a stage's k, q, beta, g by asynchronous copies; its v columns through registers (converted to 32-bit)
    constexpr int V_PER_THREAD = (TB * VB + 127) / 128;
    float v_regs[V_PER_THREAD];
    auto issue = [&](int t0, int buf) {
        const int n = min(TB, end - t0);
        for (int r = threadIdx.x; r < NG * D; r += 128) {                                 // an element of k | q (| g), for every token
            const int which = r / D, d = r - which * D;                                   // which: 0 k, 1 q, 2 the channel decays
            const float* src = which == 2 ? gch + ((size_t)t0 * H + h) * D + d : qk + ((size_t)t0 * 2 * G + (which ? 0 : G) + kvh) * D + d;
            const size_t step = which == 2 ? (size_t)H * D : (size_t)2 * G * D;
            float* dst = &ring[buf][0][which * St::KQ + (d / DP) * St::GROUP + d % DP];
            for (int tok = 0; tok < n; ++tok) cp_async4(dst + tok * St::PER_TOKEN, src + tok * step);
        }
        for (int i = threadIdx.x; i < n * 2; i += 128) {
            const int tok = i / 2, which = i % 2;                                        // 0 beta, 1 g
            cp_async4(&ring[buf][tok][NG * St::KQ + which], bg + (size_t)(t0 + tok) * 2 * H + which * H + h);
        }
#pragma unroll
        for (int e = 0; e < V_PER_THREAD; ++e) {
            const int i = threadIdx.x + e * 128, tok = i / VB, col = i % VB;
            v_regs[e] = (tok < n && j0 + col < V) ? to_float(v_in[(size_t)(t0 + tok) * v_stride + (size_t)h * V + j0 + col]) : 0.f;
        }
    };
    auto land = [&](int buf) {
        cp_async_wait_all();
#pragma unroll
        for (int e = 0; e < V_PER_THREAD; ++e) {
            const int i = threadIdx.x + e * 128, tok = i / VB, col = i % VB;
            if (tok < TB) ring[buf][tok][NG * St::KQ + 4 + col] = v_regs[e];
        }
        __syncthreads();
    };
    issue(start, 0);
    land(0);
    int buf = 0, pend_t = -1;
    float pend_out = 0.f;
    for (int t0 = start; t0 < end; t0 += TB, buf ^= 1) {
        const bool more = t0 + TB < end;
        if (more) issue(t0 + TB, buf ^ 1);
        const int n = min(TB, end - t0);
        for (int tok = 0; tok < n; ++tok) {
            const float* row = ring[buf][tok];
            float kc[DP], qc[DP], gc[CH ? DP : 1];
#pragma unroll
            for (int i = 0; i < DP; i += 4) {
                const float4 a = *reinterpret_cast<const float4*>(row + p * St::GROUP + i);
                const float4 b = *reinterpret_cast<const float4*>(row + St::KQ + p * St::GROUP + i);
                kc[i] = a.x; kc[i + 1] = a.y; kc[i + 2] = a.z; kc[i + 3] = a.w;
                qc[i] = b.x; qc[i + 1] = b.y; qc[i + 2] = b.z; qc[i + 3] = b.w;
                if (CH) {
                    const float4 c = *reinterpret_cast<const float4*>(row + 2 * St::KQ + p * St::GROUP + i);
                    gc[i] = c.x; gc[i + 1] = c.y; gc[i + 2] = c.z; gc[i + 3] = c.w;
                }
            }
            const float beta = row[NG * St::KQ], g = row[NG * St::KQ + 1], vv = row[NG * St::KQ + 4 + jl];
            // a warp issues in order: four short chains of multiply-adds instead of one long one, and the last
            // token's read-out is summed over the lanes beside this token's S^T k (two exchanges in flight at once)
            float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < DP; ++i) {
                S[i] *= CH ? gc[i] : g;
                d4[i & 3] += S[i] * kc[i];
            }
            float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
            float po = pend_out;
#pragma unroll
            for (int o = P / 2; o > 0; o >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, o);
                po += __shfl_xor_sync(0xffffffffu, po, o);
            }
            if (pend_t >= 0 && p == 0 && live) o_out[(size_t)pend_t * H * V + (size_t)h * V + j] = po;
            const float u = beta * (vv - dot);
            float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < DP; ++i) {
                S[i] += kc[i] * u;
                o4[i & 3] += S[i] * qc[i];
            }
            pend_out = (o4[0] + o4[1]) + (o4[2] + o4[3]);
            pend_t = t0 + tok;
        }
        if (more) land(buf ^ 1);
    }
    {
        float po = pend_out;                           // the last token's read-out
#pragma unroll
        for (int o = P / 2; o > 0; o >>= 1) po += __shfl_xor_sync(0xffffffffu, po, o);
        if (pend_t >= 0 && p == 0 && live) o_out[(size_t)pend_t * H * V + (size_t)h * V + j] = po;
    }
    if (write_state && live) {
#pragma unroll
        for (int i = 0; i < DP; ++i)
            if (d0 + i < D) st[(size_t)(d0 + i) * V] = S[i];
    }
}

__device__ __forceinline__ float delta_gate(float gv, int gate_act) {       // 0: silu, 1: sigmoid
    const float s = 1.f / (1.f + expf(-gv));
    return gate_act ? s : gv * s;
}

// out[t, h, :] = o[t, h, :] * rsqrt(mean(o^2) + eps) * w * act(gate[t, h, :]); one warp per (row, head)
template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ o, const float* __restrict__ w,
                                     const T* __restrict__ gate, int gate_stride, float eps, int items, int H, int V,
                                     int gate_act) {
    pdl_trigger();
    pdl_wait();
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= items) return;
    const int t = item / H, h = item % H;
    const float* src = o + (size_t)item * V;
    float ss = 0.f;
    for (int d = lane; d < V; d += 32) ss += src[d] * src[d];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)V + eps);
    const T* grow = gate + (size_t)t * gate_stride + (size_t)h * V;
    for (int d = lane; d < V; d += 32) {
        const float gv = to_float(grow[d]);
        out[(size_t)item * V + d] = from_float<T>(src[d] * inv * (w ? w[d] : 1.f) * delta_gate(gv, gate_act));
    }
}

// ---- a step of single tokens in one kernel: unit norms, beta and g, the state's update and read-out and the output
// norm for one head of one request per block (all V columns: P lanes a column, so P * V threads, at most 1024)
template <typename T, int DP, int P>
__global__ void __launch_bounds__(1024) gated_delta_single_kernel(
    T* __restrict__ out, const T* __restrict__ qkv, int qkv_stride, const T* __restrict__ b_in, int b_stride,
    const T* __restrict__ a_in, int a_stride, const T* __restrict__ gate, int gate_stride, const float* __restrict__ a_log,
    const float* __restrict__ dt_bias, const float* __restrict__ norm_w, float eps, float unit_eps, float* __restrict__ state,
    const int* __restrict__ slot_ids, int H, int G, int D, int V, int write_state, int num_slots, int* __restrict__ status,
    int channel, int gate_act) {
    extern __shared__ float sm[];                      // q [D], k [D], the decays [D], 33 for the block's sum
    float* qs = sm;
    float* ks = sm + D;
    float* gs = sm + 2 * D;
    float* red = sm + 3 * D;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, kvh = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const T* row = qkv + (size_t)t * qkv_stride;
    for (int item = warp; item < 2; item += nwarp) {                  // 0: q, 1: k of this head's q/k head
        const T* src = row + (size_t)(item * G + kvh) * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float v = to_float(src[d]);
            ss += v * v;
        }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss + unit_eps) * (item == 0 ? rsqrtf((float)D) : 1.f);
        float* dst = item == 0 ? qs : ks;
        for (int d = lane; d < D; d += 32) dst[d] = to_float(src[d]) * inv;
    }
    {
        const float rate = expf(a_log[h]);
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const int i = channel ? h * D + d : h;
            gs[d] = expf(-rate * softplus_f(to_float(a_in[(size_t)t * a_stride + i]) + dt_bias[i]));
        }
    }
    __syncthreads();
    const float beta = 1.f / (1.f + expf(-to_float(b_in[(size_t)t * b_stride + h])));
    const int p = threadIdx.x % P, d0 = p * DP;
    int j = threadIdx.x / P;
    const bool live = j < V;
    if (!live) j = V - 1;
    const int slot = zai_checked_slot(slot_ids[t], num_slots, status);
    float* st = state + (((size_t)slot * H + h) * D) * V + j;
    float S[DP];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        S[i] = d0 + i < D ? st[(size_t)(d0 + i) * V] * gs[d0 + i] : 0.f;
        dot += d0 + i < D ? S[i] * ks[d0 + i] : 0.f;
    }
#pragma unroll
    for (int o = P / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float u = beta * (to_float(row[(size_t)2 * G * D + (size_t)h * V + j]) - dot);
    float o_j = 0.f;
#pragma unroll
    for (int i = 0; i < DP; ++i) {
        if (d0 + i < D) {
            S[i] += ks[d0 + i] * u;
            o_j += S[i] * qs[d0 + i];
            if (write_state && live) st[(size_t)(d0 + i) * V] = S[i];
        }
    }
#pragma unroll
    for (int o = P / 2; o > 0; o >>= 1) o_j += __shfl_xor_sync(0xffffffffu, o_j, o);
    const float ss = block_sum((p == 0 && live) ? o_j * o_j : 0.f, red);
    const float inv = rsqrtf(ss / (float)V + eps);
    if (p == 0 && live) {
        const float gv = to_float(gate[(size_t)t * gate_stride + (size_t)h * V + j]);
        out[((size_t)t * H + h) * V + j] = from_float<T>(o_j * inv * (norm_w ? norm_w[j] : 1.f) * delta_gate(gv, gate_act));
    }
}

template <typename T, int DP, int P>
static int launch_delta_single(void* out, const void* qkv, int qkv_stride, const void* b_in, int b_stride, const void* a_in,
                               int a_stride, const void* gate, int gate_stride, const float* a_log, const float* dt_bias,
                               const float* norm_w, float eps, float unit_eps, float* state, const int* slot_ids, int B, int H, int G,
                               int D, int V, int write_state, int num_slots, int* status, int channel, int gate_act,
                               cudaStream_t stream) {
    const int threads = ((P * V + 31) / 32) * 32;
    if (threads > 1024) return ZAI_BAD_SIZE;
    return launch_pdl(gated_delta_single_kernel<T, DP, P>, dim3(B, H), dim3(threads), (size_t)(3 * D + 33) * sizeof(float), stream,
                      (T*)out, (const T*)qkv, qkv_stride, (const T*)b_in, b_stride, (const T*)a_in, a_stride, (const T*)gate,
                      gate_stride, a_log, dt_bias, norm_w, eps, unit_eps, state, slot_ids, H, G, D, V, write_state, num_slots, status,
                      channel, gate_act);
}

// 1 if a step of single tokens with these sizes can run as the one kernel above
ZAI_API int zai_gated_delta_single_supports(int D, int V) {
    const int P = D <= 128 ? 4 : 8;
    return D >= 1 && D <= 256 && V >= 1 && ((P * V + 31) / 32) * 32 <= 1024;
}

// out [B, H*V] in the model's dtype; qkv [B, qkv_stride] (q heads, k heads, v heads, after their convolutions);
// b_in [B, b_stride] (H values a row); a_in [B, a_stride] (H values a row, or H D with `channel`); gate [B, gate_stride];
// state [slots, H, D, V]; row i belongs to slot_ids[i]
ZAI_API int zai_gated_delta_single(void* out, const void* qkv, int qkv_stride, const void* b_in, int b_stride, const void* a_in,
                                   int a_stride, const void* gate, int gate_stride, int dtype, const float* a_log,
                                   const float* dt_bias, const float* norm_w, float eps, float unit_eps, float* state,
                                   const int* slot_ids, int B, int H, int G, int D, int V, int write_state, int num_slots, int* status,
                                   int channel, int gate_act, cudaStream_t stream) {
    if (B <= 0) return ZAI_OK;
    if (!zai_gated_delta_single_supports(D, V) || G < 1 || H % G != 0 || H > 65535) return ZAI_BAD_SIZE;
#define ZAI_DELTA1(DPV, PV) ZAI_DISPATCH(dtype, return launch_delta_single<T, DPV, PV>(out, qkv, qkv_stride, b_in, b_stride, a_in, a_stride, \
        gate, gate_stride, a_log, dt_bias, norm_w, eps, unit_eps, state, slot_ids, B, H, G, D, V, write_state, num_slots, status, channel, \
        gate_act, stream))
    if (D <= 16) ZAI_DELTA1(4, 4);
    if (D <= 32) ZAI_DELTA1(8, 4);
    if (D <= 64) ZAI_DELTA1(16, 4);
    if (D <= 128) ZAI_DELTA1(32, 4);
    ZAI_DELTA1(32, 8);
#undef ZAI_DELTA1
}

// gch_out null: one decay per head (into bg_out); else the decays per head and key channel [N, H, D]
ZAI_API int zai_delta_prepare(float* qk_out, float* bg_out, float* gch_out, const void* qkv, int qkv_stride, const void* b_in,
                              int b_stride, const void* a_in, int a_stride, int dtype, const float* a_log, const float* dt_bias,
                              int N, int H, int G, int D, float unit_eps, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    ZAI_DISPATCH(dtype, return launch_pdl(delta_prepare_kernel<T>, dim3(N), dim3(128), 0, stream, qk_out, bg_out, gch_out,
        (const T*)qkv, qkv_stride, (const T*)b_in, b_stride, (const T*)a_in, a_stride, a_log, dt_bias, H, G, D, unit_eps));
}

// Dynamic shared memory that keeps more than `per_sm` blocks of `kernel` off one SM.  The recurrence is a chain of
// dependent instructions per warp, so a block runs fastest with an SM's schedulers to itself; but a grid that is
// launched while the kernel before it still drains (as dependent launches are) is placed on the first SMs that have
// room, several blocks to an SM with other SMs left empty (measured: 64 blocks after a large kernel, 1130 us instead
// of 640).  Unused shared memory makes the placement even whatever runs before.
template <typename K>
static size_t delta_spread_smem(K kernel, long long blocks) {
    static int sms = 0, sm_smem = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&sm_smem, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
        if (sms < 1) sms = 1;
    }
    const long long per_sm = (blocks + sms - 1) / sms;
    if (per_sm >= 4) return 0;
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) return 0;
    // every block takes its static and dynamic bytes and 1 KB of the system's: per_sm blocks fit, per_sm + 1 do not
    const long long each = sm_smem / per_sm - 1024 - (long long)fa.sharedSizeBytes - 1024;
    const long long next = sm_smem / (per_sm + 1) - 1024 - (long long)fa.sharedSizeBytes;
    if (each <= 0 || each <= next) return 0;
    const long long dyn = each > 160 * 1024 ? 160 * 1024 : each;
    if (dyn <= next || dyn <= 0) return 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess) { cudaGetLastError(); return 0; }
    return (size_t)dyn;
}

template <typename T, int DP, int P>
static int launch_delta(float* o_out, const float* qk, const float* bg, const float* gch, const void* v_in, int v_stride,
                        float* state, const int* cu_q, const int* slot_ids, int n_seqs, int H, int G, int D, int V, int write_state,
                        int num_slots, int* status, cudaStream_t stream) {
    const int vb = 128 / P;
    const dim3 grid(n_seqs, H, (V + vb - 1) / vb);
    const long long blocks = (long long)grid.x * grid.y * grid.z;
    if (gch)
        return launch_pdl(gated_delta_kernel<T, DP, P, true>, grid, dim3(128), delta_spread_smem(gated_delta_kernel<T, DP, P, true>, blocks),
                          stream, o_out, qk, bg, gch, (const T*)v_in, v_stride, state, cu_q, slot_ids, H, G, D, V, write_state, num_slots,
                          status);
    return launch_pdl(gated_delta_kernel<T, DP, P, false>, grid, dim3(128), delta_spread_smem(gated_delta_kernel<T, DP, P, false>, blocks),
                      stream, o_out, qk, bg, gch, (const T*)v_in, v_stride, state, cu_q, slot_ids, H, G, D, V, write_state, num_slots,
                      status);
}

// o_out [N, H*V] 32-bit; qk, bg (and gch, or null) from zai_delta_prepare; v_in [N, v_stride] (heads of V values);
// state [slots, H, D, V]
ZAI_API int zai_gated_delta(float* o_out, const float* qk, const float* bg, const float* gch, const void* v_in, int v_stride,
                            int dtype, float* state, const int* cu_q, const int* slot_ids, int N, int n_seqs, int H, int G, int D,
                            int V, int write_state, int num_slots, int* status, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0) return ZAI_OK;
    if (D < 1 || D > 256 || V < 1 || G < 1 || H % G != 0 || H > 65535 || V > 65535 * 16) return ZAI_BAD_SIZE;
#define ZAI_DELTA(DPV, PV) ZAI_DISPATCH(dtype, return launch_delta<T, DPV, PV>(o_out, qk, bg, gch, v_in, v_stride, state, cu_q, \
        slot_ids, n_seqs, H, G, D, V, write_state, num_slots, status, stream))
    // four lanes a column (eight for the largest heads): measured against two and one (fewer exchanges, longer
    // chains of multiply-adds a lane), four was the fastest or level at 64-wide heads
    if (D <= 16) ZAI_DELTA(4, 4);
    if (D <= 32) ZAI_DELTA(8, 4);
    if (D <= 64) ZAI_DELTA(16, 4);
    if (D <= 128) ZAI_DELTA(32, 4);
    ZAI_DELTA(32, 8);
#undef ZAI_DELTA
}

ZAI_API int zai_gated_rmsnorm(void* out, const float* o, const float* w, const void* gate, int gate_stride, int dtype, float eps,
                              int N, int H, int V, int gate_act, cudaStream_t stream) {
    const long long items = (long long)N * H;
    if (items <= 0) return ZAI_OK;
    const long long blocks = (items + 3) / 4;
    if (blocks > 0x7fffffffLL) return ZAI_BAD_SIZE;
    ZAI_DISPATCH(dtype, return launch_pdl(gated_rmsnorm_kernel<T>, dim3((unsigned)blocks), dim3(128), 0, stream, (T*)out, o, w,
        (const T*)gate, gate_stride, eps, (int)items, H, V, gate_act));
}
