// A mixture of small gated feed-forwards: every row of the step goes to its `top` experts by router score.
//
//   z = x . Wr^T (32-bit),  s = sigmoid(z),  the `top` largest s choose the experts (ties: the lower index),
//   weights w = s of the chosen (divided by their sum with `renorm`)
//   y = sum over the chosen e of  down_e( silu(gate_e(x_e)) * up_e(x_e) ),   x_e = w_e x   (`weight_on` input)
//                                or of  w_e down_e( silu(gate_e(x)) * up_e(x) )             (`weight_on` output)
//
// Five kernels, none of which tells the host anything (the step stays a fixed list of launches):
//   * route: a block a row; the router's products summed in 32-bit in an order that depends on the width alone, the
//     choice, and the row's place among its expert's rows (a counter per expert);
//   * gather: the rows, scaled, into a layout sorted by expert in which every expert's rows start at a multiple of
//     the tile height TM (padding rows hold whatever was there: a row's result never depends on another row), and the
//     expert of every tile;
//   * two grouped products over that layout (gate|up with the activation as epilogue, then down): a block owns a
//     tile of TM rows x 64 output columns of one expert; bfloat16 on the tensor cores (mma.sync m16n8k16, cp.async
//     ring of three stages), any other case by 32-bit multiply-adds.  Steps with many rows an expert gather with a
//     tile height of 128 and run both products in the grouped mode of the tcgen05 kernel (gemm_tc.cu) instead;
//   * combine: a row's `top` results summed in 32-bit in the order of the choice and rounded once.
// A row's result depends on the row alone: on which tile it lands, what else the tile holds and in which order the
// counter was taken changes nothing, since every output element is a sum over k in a fixed order.
#include "mma_helpers.cuh"

#define MOE_TN 64          // output columns of a block
#define MOE_TK 32          // k per stage
#define MOE_ST (MOE_TK + 8)
#define MOE_STAGES 3

// Eight neighbouring values as 32-bit numbers by 16-byte accesses (the caller has checked the alignment).
__device__ __forceinline__ void moe_load8(float (&v)[8], const bf16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void moe_load8(float (&v)[8], const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void moe_store8(bf16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void moe_store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <typename T>
__device__ __forceinline__ bool moe_rows_aligned(const T* p, size_t stride, int W) {
    return (W & 7) == 0 && (stride & 7) == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// ------------------------------------------------------------------------------------------------ route
template <typename T>
__global__ void __launch_bounds__(128) moe_route_kernel(int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ rank,
                                                        int* __restrict__ counts, const T* __restrict__ x, int x_stride,
                                                        const float* __restrict__ wr, int W, int E, int top, int renorm,
                                                        int softmax) {
    extern __shared__ float sc[];                        // [E] scores
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    const T* row = x + (size_t)t * x_stride;
    // (which of the two loops runs depends on the sizes and addresses alone, never on the other rows of the step)
    const bool vec = moe_rows_aligned(x, (size_t)x_stride, W) && (reinterpret_cast<uintptr_t>(wr) & 15) == 0;
    for (int e = warp; e < E; e += 4) {
        const float* w = wr + (size_t)e * W;
        float acc = 0.f;
        if (vec) {
            for (int c = lane * 8; c < W; c += 256) {
                float xv[8], wv[8];
                moe_load8(xv, row + c);
                moe_load8(wv, w + c);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc += xv[i] * wv[i];
            }
        } else {
            for (int c = lane; c < W; c += 32) acc += to_float(row[c]) * w[c];
        }
        acc = warp_sum(acc);
        if (lane == 0) sc[e] = softmax ? acc : 1.f / (1.f + expf(-acc));
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax) {                                       // scores = softmax of the logits over all experts, in a fixed order
        float top_z = -INFINITY;
        for (int e = lane; e < E; e += 32) top_z = fmaxf(top_z, sc[e]);
        top_z = warp_max(top_z);
        float total = 0.f;
        for (int e = lane; e < E; e += 32) total += expf(sc[e] - top_z);
        total = warp_sum(total);
        for (int e = lane; e < E; e += 32) sc[e] = expf(sc[e] - top_z) / total;
        __syncwarp();
    }
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sc[e];
            if (v > best) { best = v; at = e; }          // (ascending e: the first of equals stays)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oa < at)) { best = ov; at = oa; }
        }
        if (at >= E) at = 0;                             // (scores that are no numbers: any expert, never an index outside)
        if (lane == 0) {
            ids[(size_t)t * top + k] = at;
            wts[(size_t)t * top + k] = best;
            rank[(size_t)t * top + k] = atomicAdd(&counts[at], 1);
            sc[at] = -2.f;
        }
        sum += best;
        __syncwarp();
    }
    __syncwarp();
    if (renorm && lane < top) wts[(size_t)t * top + lane] /= sum + 1e-20f;
}

// ------------------------------------------------------------------------------------------------ gather
// One block per (row, choice) and one more that writes the tiles' experts.  The first row of expert e in the sorted
// layout is sum_{e' < e} roundup(counts[e'], TM).
template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(T* __restrict__ xs, int* __restrict__ dest, int* __restrict__ tile_expert,
                                                         const T* __restrict__ x, int x_stride, const int* __restrict__ ids,
                                                         const float* __restrict__ wts, const int* __restrict__ rank,
                                                         const int* __restrict__ counts, int items, int W, int E, int top, int TM,
                                                         int max_tiles, int scale_input) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x == items) {                      // the tiles' experts (-1: a tile that no expert uses)
        __shared__ int s_tiles;
        if (threadIdx.x == 0) {
            int at = 0;
            for (int e = 0; e < E; ++e) {
                const int n = (counts[e] + TM - 1) / TM;
                for (int i = 0; i < n && at + i < max_tiles; ++i) tile_expert[at + i] = e;
                at += n;
            }
            s_tiles = at < max_tiles ? at : max_tiles;
        }
        __syncthreads();
        for (int i = s_tiles + threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
        return;
    }
    const int item = blockIdx.x, t = item / top, e = ids[item];
    float before = 0.f;                                  // (whole numbers below 2^24: exact in 32-bit floats)
    for (int o = threadIdx.x; o < e; o += blockDim.x) before += (float)(((counts[o] + TM - 1) / TM) * TM);
    const int first = (int)block_sum(before, red);
    const int d = first + rank[item];
    if (threadIdx.x == 0) dest[item] = d;
    const float w = scale_input ? wts[item] : 1.f;
    const T* src = x + (size_t)t * x_stride;
    T* dst = xs + (size_t)d * W;
    if (moe_rows_aligned(x, (size_t)x_stride, W) && (reinterpret_cast<uintptr_t>(xs) & 15) == 0) {
        for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
            float v[8];
            moe_load8(v, src + c);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = to_float(from_float<T>(v[i] * w));
            moe_store8(dst + c, v);
        }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = from_float<T>(to_float(src[c]) * w);
}

// ------------------------------------------------------------------------------------------------ grouped products
// epilogue 0: out[row, n] (TO); 1: out[row, f] = silu(gate f) * up f, the weights being [E, 2 F, K] (gate rows, up rows)
template <typename TO>
__device__ __forceinline__ void moe_store(TO* p, float v);
template <> __device__ __forceinline__ void moe_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void moe_store<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float moe_silu(float g) { return g / (1.f + expf(-g)); }
// The gated epilogues: 1  silu(g) u;  2  g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)
struct MoeAct {
    int kind;
    float limit, alpha;
    __device__ __forceinline__ float operator()(float g, float u) const {
        if (kind != 2) return moe_silu(g) * u;
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.f + expf(-alpha * g)) * (u + 1.f);
    }
};

// The weight row that row r (0..63) of a block's tile of weights holds, or -1.  Plain: output column n0 + r.  Gated:
// groups of eight rows alternate between the gate and the up rows of the same eight features.
__device__ __forceinline__ int moe_weight_row(int r, int col_block, int n_out, int gated) {
    if (!gated) {
        const int n = col_block * MOE_TN + r;
        return n < n_out ? n : -1;
    }
    const int f = col_block * (MOE_TN / 2) + (r >> 4) * 8 + (r & 7);
    return f < n_out ? ((r >> 3) & 1) * n_out + f : -1;
}

template <int TM, typename TO>
__global__ void __launch_bounds__(128) moe_gemm_mma_kernel(TO* __restrict__ out, const bf16* __restrict__ xs,
                                                           const bf16* __restrict__ w, const int* __restrict__ tile_expert,
                                                           int K, int n_out, int gated, const MoeAct act) {
    constexpr int WM = TM / 16, WN = 4 / WM, NT = 8 / WN;            // warps along rows and columns; 8-column tiles a warp
    __shared__ __align__(16) bf16 sa[MOE_STAGES][TM][MOE_ST];
    __shared__ __align__(16) bf16 sb[MOE_STAGES][MOE_TN][MOE_ST];
    pdl_trigger();
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % WM, wn = warp / WM;
    const size_t row0 = (size_t)blockIdx.x * TM;
    const bf16* wexp = w + (size_t)e * (gated ? 2 : 1) * n_out * K;
    const int n_k = (K + MOE_TK - 1) / MOE_TK;
    auto load = [&](int kt, int buf) {
        const int k0 = kt * MOE_TK;
        for (int i = tid; i < TM * (MOE_TK / 8); i += 128) {
            const int r = i / (MOE_TK / 8), c = (i % (MOE_TK / 8)) * 8;
            const bool ok = k0 + c < K;
            cp_async16(&sa[buf][r][c], xs + (row0 + r) * K + (ok ? k0 + c : 0), ok);
        }
        for (int i = tid; i < MOE_TN * (MOE_TK / 8); i += 128) {
            const int r = i / (MOE_TK / 8), c = (i % (MOE_TK / 8)) * 8;
            const int wr = moe_weight_row(r, blockIdx.y, n_out, gated);
            const bool ok = wr >= 0 && k0 + c < K;
            cp_async16(&sb[buf][r][c], wexp + (ok ? (size_t)wr * K + k0 + c : 0), ok);
        }
    };
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int s = 0; s < MOE_STAGES - 1; ++s) {
        if (s < n_k) load(s, s);
        cp_async_commit();
    }
    const int a_row = (((lane >> 3) & 1) << 3) + (lane & 7), a_dof = (lane >> 4) << 3;
    const int b_row = ((lane >> 4) << 3) + (lane & 7), b_dof = ((lane >> 3) & 1) << 3;
    for (int kt = 0; kt < n_k; ++kt) {
        cp_async_wait<MOE_STAGES - 2>();
        __syncthreads();                                 // stage kt has landed; stage kt - 1 has been read by every warp
        if (kt + MOE_STAGES - 1 < n_k) load(kt + MOE_STAGES - 1, (kt + MOE_STAGES - 1) % MOE_STAGES);
        cp_async_commit();
        const int buf = kt % MOE_STAGES;
#pragma unroll
        for (int ks = 0; ks < MOE_TK / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, &sa[buf][wm * 16 + a_row][ks * 16 + a_dof]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, &sb[buf][(wn * NT + np * 2) * 8 + b_row][ks * 16 + b_dof]);
                mma_bf16(acc[np * 2], a, b[0], b[1]);
                mma_bf16(acc[np * 2 + 1], a, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    const int g = lane >> 2, tq = lane & 3;
    const size_t ra = row0 + wm * 16 + g, rb = ra + 8;
    if (gated) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int f = blockIdx.y * (MOE_TN / 2) + (wn * (NT / 2) + np) * 8 + 2 * tq + c;
                if (f < n_out) {
                    moe_store<TO>(out + ra * n_out + f, act(acc[np * 2][c], acc[np * 2 + 1][c]));
                    moe_store<TO>(out + rb * n_out + f, act(acc[np * 2][2 + c], acc[np * 2 + 1][2 + c]));
                }
            }
        }
        return;
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int n = blockIdx.y * MOE_TN + (wn * NT + nt) * 8 + 2 * tq + c;
            if (n < n_out) {
                moe_store<TO>(out + ra * n_out + n, acc[nt][c]);
                moe_store<TO>(out + rb * n_out + n, acc[nt][2 + c]);
            }
        }
    }
}

// Any element type and any K: a tile of 16 rows x 64 columns by 32-bit multiply-adds, k in ascending order.
template <typename T, typename TO>
__global__ void __launch_bounds__(128) moe_gemm_plain_kernel(TO* __restrict__ out, const T* __restrict__ xs, const T* __restrict__ w,
                                                             const int* __restrict__ tile_expert, int K, int n_out, int gated,
                                                             const MoeAct act) {
    __shared__ float sa[16][MOE_TK + 1];
    __shared__ float sb[MOE_TN][MOE_TK + 1];
    pdl_trigger();
    pdl_wait();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int tid = threadIdx.x, r = tid >> 3, c8 = tid & 7;
    const size_t row0 = (size_t)blockIdx.x * 16;
    const T* wexp = w + (size_t)e * (gated ? 2 : 1) * n_out * K;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        __syncthreads();
        for (int i = tid; i < 16 * MOE_TK; i += 128) {
            const int rr = i / MOE_TK, kk = i % MOE_TK;
            sa[rr][kk] = k0 + kk < K ? to_float(xs[(row0 + rr) * K + k0 + kk]) : 0.f;
        }
        for (int i = tid; i < MOE_TN * MOE_TK; i += 128) {
            const int rr = i / MOE_TK, kk = i % MOE_TK;
            const int wr = moe_weight_row(rr, blockIdx.y, n_out, gated);
            sb[rr][kk] = (wr >= 0 && k0 + kk < K) ? to_float(wexp[(size_t)wr * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < MOE_TK; ++kk) {
            const float a = sa[r][kk];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(a, sb[c8 + 8 * j][kk], acc[j]);
        }
    }
    // column c8 + 8 j of the tile: gated, groups of eight alternate gate / up, so j even is a gate and j + 1 its up
    if (gated) {
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            const int f = blockIdx.y * (MOE_TN / 2) + (j / 2) * 8 + c8;
            if (f < n_out) moe_store<TO>(out + (row0 + r) * n_out + f, act(acc[j], acc[j + 1]));
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int n = blockIdx.y * MOE_TN + c8 + 8 * j;
        if (n < n_out) moe_store<TO>(out + (row0 + r) * n_out + n, acc[j]);
    }
}

// ------------------------------------------------------------------------------------------------ combine
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ y, const int* __restrict__ dest,
                                   const float* __restrict__ wts, int W, int top, int scale_output) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if ((W & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {      // the same sums in the same order, eight columns at a time
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int k = 0; k < top; ++k) {
                float v[8];
                moe_load8(v, y + (size_t)dest[(size_t)t * top + k] * W + c);
                const float wk = scale_output ? wts[(size_t)t * top + k] : 1.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += scale_output ? v[i] * wk : v[i];
            }
            moe_store8(out + (size_t)t * W + c, acc);
        }
        return;
    }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const float v = y[(size_t)dest[(size_t)t * top + k] * W + c];
            acc += scale_output ? v * wts[(size_t)t * top + k] : v;
        }
        out[(size_t)t * W + c] = from_float<T>(acc);
    }
}

// ------------------------------------------------------------------------------------------------ launchers
// ids, rank [N, top] int; wts [N, top] 32-bit; counts [E] int, zeroed here; x [N, x_stride] in `dtype`; wr [E, W] 32-bit
ZAI_API int zai_moe_route(int* ids, float* wts, int* rank, int* counts, const void* x, int x_stride, int dtype, const float* wr,
                          int N, int W, int E, int top, int renorm, int softmax, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (E < 1 || top < 1 || top > E || top > 32 || E > 8192 || W < 1) return ZAI_BAD_SIZE;
    cudaError_t rc = cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int), stream);
    if (rc != cudaSuccess) return (int)rc;
    ZAI_DISPATCH(dtype, return launch_pdl(moe_route_kernel<T>, dim3(N), dim3(128), (size_t)E * sizeof(float), stream, ids, wts, rank,
                                          counts, (const T*)x, x_stride, wr, W, E, top, renorm, softmax));
}

// The most tiles of TM rows that N x top choices over E experts can take.
ZAI_API int zai_moe_max_tiles(int N, int top, int E, int TM) {
    const long long items = (long long)N * top;
    const long long t = items / TM + (items < E ? items : E);
    return t > 0x7fffffff ? -1 : (int)t;
}

// xs [max_tiles * TM, W] in `dtype`; dest [N, top]; tile_expert [max_tiles]
ZAI_API int zai_moe_gather(void* xs, int* dest, int* tile_expert, const void* x, int x_stride, int dtype, const int* ids,
                           const float* wts, const int* rank, const int* counts, int N, int W, int E, int top, int TM, int max_tiles,
                           int scale_input, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    const long long items = (long long)N * top;
    if (items >= 0x7fffffff || (TM != 16 && TM != 64 && TM != 128) || (long long)max_tiles * TM >= (1 << 24)) return ZAI_BAD_SIZE;
    ZAI_DISPATCH(dtype, return launch_pdl(moe_gather_kernel<T>, dim3((unsigned)items + 1), dim3(128), 0, stream, (T*)xs, dest,
                                          tile_expert, (const T*)x, x_stride, ids, wts, rank, counts, (int)items, W, E, top, TM,
                                          max_tiles, scale_input));
}

// out [max_tiles * TM, n_out] (32-bit if out_f32, else `dtype`) = xs [max_tiles * TM, K] . w[expert of the tile]^T;
// w [E, n_out, K], or with `gated` [E, 2 n_out, K] and out = silu(gate) * up (gated 1) or the bounded gated activation with
// `limit` and `alpha` (gated 2).  TM 16 or 64 (the gather's).
ZAI_API int zai_moe_gemm(void* out, int out_f32, const void* xs, const void* w, int dtype, const int* tile_expert, int max_tiles,
                         int TM, int K, int n_out, int gated, float limit, float alpha, cudaStream_t stream) {
    if (max_tiles <= 0) return ZAI_OK;
    const MoeAct act = {gated, limit, alpha};
    if (K < 1 || n_out < 1 || (TM != 16 && TM != 64)) return ZAI_BAD_SIZE;
    const int cols = gated ? MOE_TN / 2 : MOE_TN;
    const dim3 grid(max_tiles, (n_out + cols - 1) / cols);
    if (grid.y > 65535) return ZAI_BAD_SIZE;
    if (dtype == ZAI_BF16 && K % 8 == 0) {
#define MOE_GO(TMV, TOV) return launch_pdl(moe_gemm_mma_kernel<TMV, TOV>, grid, dim3(128), 0, stream, (TOV*)out, (const bf16*)xs, \
                                           (const bf16*)w, tile_expert, K, n_out, gated, act)
        if (TM == 16) { if (out_f32) MOE_GO(16, float); else MOE_GO(16, bf16); }
        if (out_f32) MOE_GO(64, float); else MOE_GO(64, bf16);
#undef MOE_GO
    }
    if (TM != 16) return ZAI_BAD_SIZE;                   // the plain kernel's tiles are 16 rows high
    if (dtype == ZAI_BF16) {
        if (out_f32) return launch_pdl(moe_gemm_plain_kernel<bf16, float>, grid, dim3(128), 0, stream, (float*)out, (const bf16*)xs,
                                       (const bf16*)w, tile_expert, K, n_out, gated, act);
        return launch_pdl(moe_gemm_plain_kernel<bf16, bf16>, grid, dim3(128), 0, stream, (bf16*)out, (const bf16*)xs, (const bf16*)w,
                          tile_expert, K, n_out, gated, act);
    }
    if (dtype != ZAI_F32) return ZAI_BAD_DTYPE;
    return launch_pdl(moe_gemm_plain_kernel<float, float>, grid, dim3(128), 0, stream, (float*)out, (const float*)xs, (const float*)w,
                      tile_expert, K, n_out, gated, act);
}

// out [N, W] in `dtype` = sum over a row's choices of y[dest], times the choice's weight with `scale_output`
ZAI_API int zai_moe_combine(void* out, int dtype, const float* y, const int* dest, const float* wts, int N, int W, int top,
                            int scale_output, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    ZAI_DISPATCH(dtype, return launch_pdl(moe_combine_kernel<T>, dim3(N), dim3(W >= 1024 ? 256 : 128), 0, stream, (T*)out, y, dest,
                                          wts, W, top, scale_output));
}
