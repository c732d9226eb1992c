// A matrix memory with exponential gates kept in logarithms (the mLSTM cell of the xLSTM family), per request and head:
//
//   i_t = cap tanh((x_i + b_i) / cap),   f_t = logsigmoid(cap tanh((x_f + b_f) / cap))          log gates, one pair a head
//   m_t = max(f_t + m_(t-1), i_t)                                                                   running maximum, m_(-1) = 0
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),   q_t = x_q D^(-1/2)
//   out = o / rms(o) per head * weight * sigmoid(gate)
//
// The normaliser n is one more column of S (the column of a value that is always 1), and every column carries its own
// copy of m in a row behind its D rows: the kept state is [heads, D + 1, Dv + 1], 32-bit, and a column's walk needs
// nothing from another column.  `mlstm_scan_kernel`: a warp owns 32 columns of one head of one request and walks the
// request's rows of the step in order, its column of S in registers, the rows' q, k and gates staged in shared memory a
// tile of rows at a time by a second warp (the next tile comes in while a tile is walked); it leaves S^T q per column,
// n . q and m per row.  `mlstm_output_kernel` divides, norms and gates.
// Gates, decays, the state and the sums are 32-bit in both modes; a row's result depends on the request's rows alone and
// is the same whether they come as one portion, as several or one by one.
#include "common.cuh"

// Rows staged at a time: as many as make the staged q and k 2 x 1024 values, at most 32 (a lane computes one row's gates).
template <int DMAX> struct MlstmTile { static constexpr int TT = 1024 / DMAX < 32 ? 1024 / DMAX : 32; };

__device__ __forceinline__ float mlstm_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// Two warps a block: warp 1 brings the rows of the next tile from memory into one of two shared buffers (q scaled, k, the
// lanes' values, the two log gates, all as 32-bit numbers; zeros beyond D and beyond the span) while warp 0, which owns the 32
// columns, walks the tile before; they meet at one barrier a tile.
template <typename T, int DMAX>
__global__ void __launch_bounds__(64) mlstm_scan_kernel(
    float* __restrict__ part, const T* __restrict__ y, int y_stride, int q_at, int k_at, int v_at, int i_at, int f_at,
    const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, float* __restrict__ state,
    const int* __restrict__ cu_q, const int* __restrict__ slot_ids, int num_slots, int* __restrict__ status, int H, int D, int Dv,
    int write_state) {
    constexpr int TT = MlstmTile<DMAX>::TT, PER = TT * DMAX / 32;      // staged values of q (and of k) a lane brings
    __shared__ __align__(16) float sq[2][TT * DMAX], sk[2][TT * DMAX], sv[2][TT * 32], sg[2][TT * 2];
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.z * 32 + lane;         // this lane's column; column Dv is the normaliser
    const bool live = c <= Dv;
    const int r0 = cu_q[s], r1 = cu_q[s + 1];
    if (r1 <= r0) return;
    const int n_tiles = (r1 - r0 + TT - 1) / TT;

    if (warp == 1) {                              // ---- the rows' way into shared memory
        const float qscale = rsqrtf((float)D);
        const float bi = bias_i[h], bf = bias_f[h];
        for (int n = 0; n < n_tiles; ++n) {
            const int t0 = r0 + n * TT, nt = min(TT, r1 - t0), buf = n & 1;
            // all of the tile's loads are issued before any of them is used: one trip to memory a tile, not one a batch
            T fq[PER], fk[PER], fv[TT];
            float gate_i = 0.f, gate_f = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = lane + 32 * i, tt = e / DMAX, d = e % DMAX;
                const bool ok = tt < nt && d < D;
                const T* row = y + (size_t)(t0 + (ok ? tt : 0)) * y_stride + h * D + (ok ? d : 0);
                fq[i] = ok ? row[q_at] : from_float<T>(0.f);
                fk[i] = ok ? row[k_at] : from_float<T>(0.f);
            }
#pragma unroll
            for (int tt = 0; tt < TT; ++tt)
                fv[tt] = (tt < nt && c < Dv) ? y[(size_t)(t0 + tt) * y_stride + v_at + h * Dv + c] : from_float<T>(1.f);
            if (lane < nt) {
                const T* row = y + (size_t)(t0 + lane) * y_stride;
                gate_i = to_float(row[i_at + h]);
                gate_f = to_float(row[f_at + h]);
            }
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                sq[buf][lane + 32 * i] = to_float(fq[i]) * qscale;
                sk[buf][lane + 32 * i] = to_float(fk[i]);
            }
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) sv[buf][tt * 32 + lane] = to_float(fv[tt]);
            if (lane < nt) {
                sg[buf][2 * lane] = cap * tanhf((gate_i + bi) / cap);
                sg[buf][2 * lane + 1] = mlstm_logsigmoid(cap * tanhf((gate_f + bf) / cap));
            }
            __syncthreads();                      // tile n is there; tile n - 1 has been walked (its buffer is filled next)
        }
        __syncthreads();
        return;
    }

    // ---- the walk
    const int slot = zai_checked_slot(slot_ids[s], num_slots, status);
    float* st = state + (((size_t)slot * H + h) * (D + 1)) * (Dv + 1);
    float col[DMAX];
#pragma unroll
    for (int d = 0; d < DMAX; ++d) col[d] = (live && d < D) ? st[(size_t)d * (Dv + 1) + c] : 0.f;
    float m = live ? st[(size_t)D * (Dv + 1) + c] : 0.f;
    __syncthreads();                              // tile 0 is there
    for (int n = 0; n < n_tiles; ++n) {
        const int t0 = r0 + n * TT, nt = min(TT, r1 - t0), buf = n & 1;
        for (int tt = 0; tt < nt; ++tt) {
            const float gi = sg[buf][2 * tt], gf = sg[buf][2 * tt + 1];
            const float m_new = fmaxf(gf + m, gi);
            const float keep = expf(gf + m - m_new), take = expf(gi - m_new) * sv[buf][tt * 32 + lane];
            const float* qr = sq[buf] + tt * DMAX;
            const float* kr = sk[buf] + tt * DMAX;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            // (beyond D the staged q and k are zeros and the column stays zero: no bound is checked)
#pragma unroll
            for (int d = 0; d < DMAX; d += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kr + d), q4 = *reinterpret_cast<const float4*>(qr + d);
                col[d] = fmaf(keep, col[d], take * k4.x);
                col[d + 1] = fmaf(keep, col[d + 1], take * k4.y);
                col[d + 2] = fmaf(keep, col[d + 2], take * k4.z);
                col[d + 3] = fmaf(keep, col[d + 3], take * k4.w);
                a0 = fmaf(col[d], q4.x, a0);
                a1 = fmaf(col[d + 1], q4.y, a1);
                a2 = fmaf(col[d + 2], q4.z, a2);
                a3 = fmaf(col[d + 3], q4.w, a3);
            }
            m = m_new;
            if (live) {
                float* o = part + ((size_t)(t0 + tt) * H + h) * (Dv + 2);
                o[c] = (a0 + a1) + (a2 + a3);
                if (c == Dv) o[Dv + 1] = m_new;
            }
        }
        __syncthreads();                          // this tile's buffer may be filled again; the next tile is there
    }
    if (write_state && live) {
#pragma unroll
        for (int d = 0; d < DMAX; ++d)
            if (d < D) st[(size_t)d * (Dv + 1) + c] = col[d];
        st[(size_t)D * (Dv + 1) + c] = m;
    }
}

// part [N, H, Dv + 2]: S^T q per column, then n . q, then m.  One block a row, a warp a head at a time.
template <typename T>
__global__ void __launch_bounds__(128) mlstm_output_kernel(T* __restrict__ out, const float* __restrict__ part, const T* __restrict__ gate,
                                                           int gate_stride, const float* __restrict__ weight, float eps, int H, int Dv) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarp) {
        const float* p = part + ((size_t)t * H + h) * (Dv + 2);
        const float den = fmaxf(fabsf(p[Dv]), expf(-p[Dv + 1])) + 1e-6f;
        float ss = 0.f;
        for (int c = lane; c < Dv; c += 32) {
            const float o = p[c] / den;
            ss += o * o;
        }
        const float inv = rsqrtf(warp_sum(ss) / (float)Dv + eps);
        for (int c = lane; c < Dv; c += 32) {
            const float g = to_float(gate[(size_t)t * gate_stride + h * Dv + c]);
            out[((size_t)t * H + h) * Dv + c] = from_float<T>(p[c] / den * inv * weight[h * Dv + c] / (1.f + expf(-g)));
        }
    }
}

// y [N, y_stride]: the stacked projections, with q (H D), k (H D), v (H Dv), the gate (H Dv) and the two log gates' inputs (H
// each) starting at the given columns.  state [num_slots, H, D + 1, Dv + 1] 32-bit; part [N, H, Dv + 2] 32-bit scratch;
// out [N, H Dv].
ZAI_API int zai_mlstm(void* out, float* part, const void* y, int y_stride, int dtype, int q_at, int k_at, int v_at, int g_at, int i_at,
                      int f_at, const float* bias_i, const float* bias_f, float cap, const float* weight, float eps, float* state,
                      const int* cu_q, const int* slot_ids, int num_slots, int* status, int N, int S, int H, int D, int Dv,
                      int write_state, cudaStream_t stream) {
    if (N <= 0 || S <= 0) return ZAI_OK;
    if (H < 1 || H > 65535 || D < 1 || D > 256 || Dv < 1 || cap <= 0.f) return ZAI_BAD_SIZE;
    const dim3 grid(S, H, (Dv + 1 + 31) / 32);
    int rc;
#define MLSTM_GO(DM) ZAI_DISPATCH(dtype, rc = launch_pdl(mlstm_scan_kernel<T, DM>, grid, dim3(64), 0, stream, part, (const T*)y, \
        y_stride, q_at, k_at, v_at, i_at, f_at, bias_i, bias_f, cap, state, cu_q, slot_ids, num_slots, status, H, D, Dv, write_state))
    if (D <= 16) MLSTM_GO(16);
    else if (D <= 32) MLSTM_GO(32);
    else if (D <= 64) MLSTM_GO(64);
    else if (D <= 128) MLSTM_GO(128);
    else MLSTM_GO(256);
#undef MLSTM_GO
    if (rc != 0) return rc;
    ZAI_DISPATCH(dtype, return launch_pdl(mlstm_output_kernel<T>, dim3(N), dim3(128), 0, stream, (T*)out, part, (const T*)y + g_at,
                                          y_stride, weight, eps, H, Dv));
}
