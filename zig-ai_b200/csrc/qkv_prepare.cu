// Between a stacked projection and attention, for mixers whose q and k are normed over the whole projection
// or per head, rotated from a table, and whose heads may be wider in the cache than in the projection:
//
//   zai_qkv_prepare     y = [q (Hq D) | k (Hkv D) | v (Hkv Dv) | ...] per row:
//                       q, k <- x * rsqrt(mean(x^2) + eps) * gamma   over the whole of q (of k), per head, or not at all
//                       pairs (x[i], x[i + rot/2]), i < rot/2, of every head turn by the row's (cos, sin) table
//                       q -> [N, Hq, Dp],  k, v -> pages[page(pos), 0|1, kv head, pos % page_size, :Dp]
//                       (Dp >= D, Dv: zeros behind a head's own values; zeros change neither a score nor a sum)
//                       optionally the queries times 1 + coef * ln(floor((pos + 1) / every) + 1), and the cached values
//                       (1 - lambda) v + lambda v_first with an earlier layer's values of the same rows
//   zai_latent_prepare  the rotated parts of the queries of latent attention, and per row the normed latent and the
//                       rotated shared key part into pages[page(pos), pos % page_size, :rank + rot]
//   zai_sigmoid_gate    out = o * sigmoid(gate), the gate one number per head or per element
//
// Norms, rotations and sigmoids are 32-bit; what is stored is rounded once to the model's dtype.  One block per row;
// the order of every reduction depends only on the sizes, so a row's result does not depend on its batch.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(
    const T* __restrict__ y, int y_stride, const float* __restrict__ q_gamma, const float* __restrict__ k_gamma, float eps,
    int scope, const float2* __restrict__ cs_table, int rot, const int* __restrict__ positions, const int* __restrict__ seq_idx,
    const int* __restrict__ block_table, int table_width, T* __restrict__ pages, int page_size, T* __restrict__ q_out,
    int Hq, int Hkv, int D, int Dv, int Dp, int write, int num_pages, int* __restrict__ status, float temp_coef, int temp_every,
    const T* __restrict__ v_first, int v_first_stride, const float* __restrict__ v_lambda) {
    extern __shared__ float smem[];
    __shared__ float red[33];
    const int half = rot / 2;
    const int nq = Hq * D, nk = Hkv * D;
    float* buf = smem;                      // [nq + nk] q then k, 32-bit
    float* cs = smem + nq + nk;             // [half] cos
    float* sn = cs + half;                  // [half] sin
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = y + (size_t)t * y_stride;
    for (int i = tid; i < half; i += blockDim.x) {
        const float2 v = cs_table[(size_t)t * half + i];
        cs[i] = v.x;
        sn[i] = v.y;
    }
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < nq + nk; i += blockDim.x) {
        const float v = to_float(row[i]);
        buf[i] = v;
        if (i < nq) sq += v * v; else sk += v * v;
    }
    if (scope == 2) {
        const float inv_q = rsqrtf(block_sum(sq, red) / (float)nq + eps);
        const float inv_k = rsqrtf(block_sum(sk, red) / (float)nk + eps);
        for (int i = tid; i < nq + nk; i += blockDim.x)
            buf[i] *= i < nq ? inv_q * q_gamma[i] : inv_k * k_gamma[i - nq];
    } else if (scope == 1) {
        __syncthreads();
        for (int h = warp; h < Hq + Hkv; h += nwarp) {
            float* x = buf + (size_t)h * D;
            const float* gamma = h < Hq ? q_gamma : k_gamma;
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss += x[d] * x[d];
            const float inv = rsqrtf(warp_sum(ss) / (float)D + eps);
            for (int d = lane; d < D; d += 32) x[d] *= inv * gamma[d];
        }
    }
    __syncthreads();
    // rotated (or passed through) and padded to Dp: element d of head h
    auto turned = [&](const float* x, int d) -> float {
        if (d < half) return x[d] * cs[d] - x[d + half] * sn[d];
        if (d < rot) return x[d - half] * sn[d - half] + x[d] * cs[d - half];
        return d < D ? x[d] : 0.f;
    };
    const int pos = positions[t];
    // the queries' temperature: 1 + coef * ln(floor((pos + 1) / every) + 1), a step function of the position
    const float temp = temp_every > 0 ? 1.f + temp_coef * logf((float)((pos < 0 ? 0 : pos + 1) / temp_every + 1)) : 1.f;
    T* qrow = q_out + (size_t)t * Hq * Dp;
    for (int i = tid; i < Hq * Dp; i += blockDim.x) {
        const int h = i / Dp, d = i - h * Dp;
        qrow[i] = from_float<T>(turned(buf + (size_t)h * D, d) * temp);
    }
    if (!write) return;
    const int page = zai_checked_page(block_table + (size_t)seq_idx[t] * table_width, table_width,
                                      pos < 0 ? -1 : pos / page_size, num_pages, status);
    const int off = pos < 0 ? 0 : pos % page_size;
    T* kpage = pages + (size_t)page * 2 * Hkv * page_size * Dp;
    T* vpage = kpage + (size_t)Hkv * page_size * Dp;
    const T* vrow = row + nq + nk;
    // values mixed with an earlier layer's values of the same token: (1 - lambda) v + lambda v_first, in 32-bit
    const T* frow = v_first ? v_first + (size_t)t * v_first_stride : nullptr;
    const float lam = frow ? v_lambda[0] : 0.f;
    for (int i = tid; i < Hkv * Dp; i += blockDim.x) {
        const int g = i / Dp, d = i - g * Dp;
        const size_t at = ((size_t)g * page_size + off) * Dp + d;
        kpage[at] = from_float<T>(turned(buf + nq + (size_t)g * D, d));
        if (d >= Dv) vpage[at] = from_float<T>(0.f);
        else if (!frow) vpage[at] = vrow[(size_t)g * Dv + d];
        else vpage[at] = from_float<T>((1.f - lam) * to_float(vrow[(size_t)g * Dv + d]) + lam * to_float(frow[(size_t)g * Dv + d]));
    }
}

ZAI_API int zai_qkv_prepare(const void* y, int y_stride, int dtype, const float* q_gamma, const float* k_gamma, float eps, int scope,
                            const float2* cs_table, int rot, const int* positions, const int* seq_idx, const int* block_table,
                            int table_width, void* pages, int page_size, void* q_out, int N, int Hq, int Hkv, int D, int Dv,
                            int Dp, int write, int num_pages, int* status, float temp_coef, int temp_every, const void* v_first,
                            int v_first_stride, const float* v_lambda, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (Hq < 1 || Hkv < 1 || D < 1 || Dv < 1 || Dp < D || Dp < Dv || rot < 0 || rot > D || rot % 2 || scope < 0 || scope > 2
        || (scope && (!q_gamma || !k_gamma)) || (rot && !cs_table) || temp_every < 0 || (v_first && !v_lambda))
        return ZAI_BAD_SIZE;
    const size_t smem = ((size_t)(Hq + Hkv) * D + rot) * sizeof(float);
    if (smem > 200 * 1024) return ZAI_BAD_SIZE;
    static unsigned long long done_f32 = 0, done_bf16 = 0;
    if (smem > 48 * 1024) {
        if (dtype == ZAI_F32 && zai_first_on_device(&done_f32))
            cudaFuncSetAttribute(qkv_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (dtype == ZAI_BF16 && zai_first_on_device(&done_bf16))
            cudaFuncSetAttribute(qkv_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    ZAI_DISPATCH(dtype, return launch_pdl(qkv_prepare_kernel<T>, dim3(N), dim3(256), smem, stream, (const T*)y, y_stride, q_gamma,
                                          k_gamma, eps, scope, cs_table, rot, positions, seq_idx, block_table, table_width, (T*)pages,
                                          page_size, (T*)q_out, Hq, Hkv, D, Dv, Dp, write, num_pages, status, temp_coef, temp_every,
                                          (const T*)v_first, v_first_stride, v_lambda));
    return launch_status();
}

// q [N, H, D + Dr] (row stride q_stride): its rotated parts -> q_rot [N, H, Dr].  dkv [N, R + Dr] (row stride dkv_stride, may be
// null): c = rms(dkv[:R]) * gamma, r = rotate(dkv[R:]) -> pages[page(pos), pos % page_size, :R + Dr].
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ dkv, int dkv_stride, const float* __restrict__ gamma, float eps,
    const float2* __restrict__ cs_table, const int* __restrict__ positions, const int* __restrict__ seq_idx,
    const int* __restrict__ block_table, int table_width, T* __restrict__ pages, int page_size, T* __restrict__ q_rot,
    int H, int D, int Dr, int R, int num_pages, int* __restrict__ status) {
    extern __shared__ float smem[];
    __shared__ float red[33];
    const int half = Dr / 2;
    float* cs = smem;                       // [half]
    float* sn = smem + half;                // [half]
    const int tid = threadIdx.x;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = tid; i < half; i += blockDim.x) {
        const float2 v = cs_table[(size_t)t * half + i];
        cs[i] = v.x;
        sn[i] = v.y;
    }
    __syncthreads();
    const T* qrow = q + (size_t)t * q_stride;
    T* orow = q_rot + (size_t)t * H * Dr;
    for (int i = tid; i < H * half; i += blockDim.x) {
        const int h = i / half, d = i - h * half;
        const T* x = qrow + (size_t)h * (D + Dr) + D;
        const float a = to_float(x[d]), b = to_float(x[d + half]);
        orow[(size_t)h * Dr + d] = from_float<T>(a * cs[d] - b * sn[d]);
        orow[(size_t)h * Dr + d + half] = from_float<T>(b * cs[d] + a * sn[d]);
    }
    if (!dkv) return;
    const T* drow = dkv + (size_t)t * dkv_stride;
    float ss = 0.f;
    for (int i = tid; i < R; i += blockDim.x) {
        const float v = to_float(drow[i]);
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)R + eps);
    const int pos = positions[t];
    const int page = zai_checked_page(block_table + (size_t)seq_idx[t] * table_width, table_width,
                                      pos < 0 ? -1 : pos / page_size, num_pages, status);
    const int off = pos < 0 ? 0 : pos % page_size;
    T* dst = pages + ((size_t)page * page_size + off) * (R + Dr);
    for (int i = tid; i < R; i += blockDim.x) dst[i] = from_float<T>(to_float(drow[i]) * inv * gamma[i]);
    for (int d = tid; d < half; d += blockDim.x) {
        const float a = to_float(drow[R + d]), b = to_float(drow[R + d + half]);
        dst[R + d] = from_float<T>(a * cs[d] - b * sn[d]);
        dst[R + d + half] = from_float<T>(b * cs[d] + a * sn[d]);
    }
}

ZAI_API int zai_latent_prepare(const void* q, int q_stride, const void* dkv, int dkv_stride, int dtype, const float* gamma, float eps,
                               const float2* cs_table, const int* positions, const int* seq_idx, const int* block_table,
                               int table_width, void* pages, int page_size, void* q_rot, int N, int H, int D, int Dr, int R,
                               int num_pages, int* status, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (H < 1 || D < 0 || Dr < 2 || Dr % 2 || R < 1 || !cs_table || (dkv && !gamma) || Dr > 8192) return ZAI_BAD_SIZE;
    ZAI_DISPATCH(dtype, return launch_pdl(latent_prepare_kernel<T>, dim3(N), dim3(256), (size_t)Dr * sizeof(float), stream,
                                          (const T*)q, q_stride, (const T*)dkv, dkv_stride, gamma, eps, cs_table, positions, seq_idx,
                                          block_table, table_width, (T*)pages, page_size, (T*)q_rot, H, D, Dr, R, num_pages, status));
    return launch_status();
}

// out[n, h, d] = in[n * in_row + h * in_head + d] * sigmoid(gate[n * gate_stride + (per_head ? h : h * Dh + d)])
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ in, long long in_row, long long in_head,
                                    const T* __restrict__ gate, int gate_stride, int per_head, long long total, int H, int Dh) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int d = (int)(i % Dh);
    const long long nh = i / Dh;
    const int h = (int)(nh % H);
    const long long n = nh / H;
    const float g = to_float(gate[n * gate_stride + (per_head ? h : h * Dh + d)]);
    const float v = to_float(in[n * in_row + h * in_head + d]);
    out[i] = from_float<T>(v / (1.f + expf(-g)));
}

ZAI_API int zai_sigmoid_gate(void* out, const void* in, long long in_row, long long in_head, const void* gate, int gate_stride,
                             int dtype, int per_head, int N, int H, int Dh, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (H < 1 || Dh < 1) return ZAI_BAD_SIZE;
    const long long total = (long long)N * H * Dh;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    ZAI_DISPATCH(dtype, return launch_pdl(sigmoid_gate_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)in, in_row,
                                          in_head, (const T*)gate, gate_stride, per_head, total, H, Dh));
    return launch_status();
}
