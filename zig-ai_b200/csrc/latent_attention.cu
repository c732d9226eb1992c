// Causal attention of many heads over one shared cached vector per position (latent attention with the key and
// value expansions folded into the query and the output):
//
//   cached row j = [c_j (R values) | r_j (Dr values)]          pages [num_pages, page_size, R + Dr]
//   s_j = (q_lat . c_j + q_rot . r_j) * scale                  for cached positions j <= pos, same request
//   o   = sum_j softmax(s)_j c_j                               [R] per row and head
//
// With `sink` (one 32-bit number per head) the softmax's denominator holds one more term, exp(sink_h): it has no
// key and no value, is not scaled, and counts once for a row whatever the number of key ranges.
//
// A block owns one row of the step and up to LA_WARPS heads (one warp a head).  The cached rows are brought into
// shared memory 32 at a time, once for all heads of the block, as 32-bit values; lane j of every warp scores key j
// (rows are padded by one word, so the lanes read different banks), the warp keeps an online softmax, and every lane
// sums its share of the output dimensions.  Scores, weights and sums are 32-bit.  Keys are always visited from
// position 0 in steps of 32, so a row's result does not depend on how the request was cut into steps or on its batch.
#include "mma_helpers.cuh"

#define LA_WARPS 8
#define LA_KEYS 32

template <typename T, int MAXR>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(
    T* __restrict__ out, const T* __restrict__ q_lat, const T* __restrict__ q_rot, const T* __restrict__ pages,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ positions, const int* __restrict__ seq_idx,
    int page_size, int H, int R, int Dr, float scale, int num_pages, int* __restrict__ status, const float* __restrict__ sink) {
    extern __shared__ float smem[];
    const int W = R + Dr, WP = W + 1;
    float* qs = smem;                                   // [LA_WARPS][W]  the block's queries, scaled
    float* ks = smem + (size_t)LA_WARPS * W;            // [LA_KEYS][WP]  a tile of cached rows
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y * LA_WARPS + warp;
    const bool live = h < H;
    const int pos = positions[t];
    const ZaiTableRow table{block_table + (size_t)seq_idx[t] * table_width, table_width, num_pages, status};
    if (live) {
        const T* a = q_lat + ((size_t)t * H + h) * R;
        const T* b = q_rot + ((size_t)t * H + h) * Dr;
        float* q = qs + (size_t)warp * W;
        for (int d = lane; d < R; d += 32) q[d] = to_float(a[d]) * scale;
        for (int d = lane; d < Dr; d += 32) q[R + d] = to_float(b[d]) * scale;
    }
    const int kend = pos + 1;
    float m = -INFINITY, l = 0.f;
    float acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
    for (int base = 0; base < kend; base += LA_KEYS) {
        const int n = min(LA_KEYS, kend - base);
        __syncthreads();                                // the tile before this one has been read by every warp
        for (int j = warp; j < n; j += LA_WARPS) {
            const int key = base + j;
            const int page = table.page(key / page_size);
            const T* src = pages + ((size_t)page * page_size + key % page_size) * W;
            float* dst = ks + (size_t)j * WP;
            for (int d = lane; d < W; d += 32) dst[d] = to_float(src[d]);
        }
        __syncthreads();
        if (!live) continue;
        const float* q = qs + (size_t)warp * W;
        float s = -INFINITY;
        if (lane < n) {
            const float* k = ks + (size_t)lane * WP;
            float d0 = 0.f, d1 = 0.f;
            int d = 0;
            for (; d + 1 < W; d += 2) {
                d0 += q[d] * k[d];
                d1 += q[d + 1] * k[d + 1];
            }
            if (d < W) d0 += q[d] * k[d];
            s = d0 + d1;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = lane < n ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);             // m = -inf at first: 0
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] *= corr;
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* v = ks + (size_t)jj * WP;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                const int d = lane + 32 * r;
                if (d < R) acc[r] += pj * v[d];
            }
        }
        m = m_new;
    }
    if (!live) return;
    if (sink) {                                          // one more term of the denominator
        const float sk = sink[h], m_new = fmaxf(m, sk), corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] *= corr;
    }
    const float inv = 1.f / l;
    T* orow = out + ((size_t)t * H + h) * R;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < R) orow[d] = from_float<T>(acc[r] * inv);
    }
}

template <typename T, int MAXR>
static int launch_latent(void* out, const void* q_lat, const void* q_rot, const void* pages, const int* block_table, int table_width,
                         const int* positions, const int* seq_idx, int page_size, int N, int H, int R, int Dr, float scale,
                         int num_pages, int* status, const float* sink, cudaStream_t stream) {
    const int W = R + Dr;
    const size_t smem = ((size_t)LA_WARPS * W + (size_t)LA_KEYS * (W + 1)) * sizeof(float);
    static unsigned long long done = 0;
    if (smem > 48 * 1024 && zai_first_on_device(&done))
        cudaFuncSetAttribute(latent_attention_kernel<T, MAXR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return launch_pdl(latent_attention_kernel<T, MAXR>, dim3(N, (H + LA_WARPS - 1) / LA_WARPS), dim3(LA_WARPS * 32), smem, stream,
                      (T*)out, (const T*)q_lat, (const T*)q_rot, (const T*)pages, block_table, table_width, positions, seq_idx,
                      page_size, H, R, Dr, scale, num_pages, status, sink);
}

// ------------------------------------------------------------------------------------------ tensor cores (bfloat16)
// A warp owns one row of the step, 16 of its heads (the 16 rows of an m16n8k16 product), one block of up to 128
// output columns and one range of `split_keys` keys.  Per tile of 32 cached rows, brought into the warp's own part
// of shared memory by cp.async (two buffers): S = Q K^T over all R + Dr dimensions, the online softmax in 32-bit
// (base 2), and O += P V with the tile's first R columns as V, P rounded to bfloat16 as the product's operand.
// Warps never wait for one another.  With R > 128 every block of output columns computes S again (S is
// (R + Dr) / 16 steps for 4 key groups, O 2 steps for 16 column groups: 1.5 times the work at R = 256, Dr = 32).
// With several key ranges a warp leaves its unnormalised O, its maximum and its sum in scratch, and a second
// kernel adds the ranges up in order; which range a key belongs to depends on its position alone.
#define LM_KT 32           // keys per tile

// A tile of LM_KT cached rows into shared memory: four lanes share a row (64 consecutive bytes an instruction); a lane
// looks its four rows' pages up first, all at once, and then only issues copies.
__device__ __forceinline__ void lm_load_tile(bf16* dst, int ST, const bf16* __restrict__ pages, const ZaiTableRow& table, int t0,
                                             int khi, int page_size, int W, int lane) {
    const int CH = W / 8;
    const bf16* src[LM_KT / 8];
#pragma unroll
    for (int k = 0; k < LM_KT / 8; ++k) {
        const int j = t0 + (lane >> 2) + 8 * k;
        src[k] = j < khi ? pages + ((size_t)table.page(j / page_size) * page_size + j % page_size) * W : nullptr;
    }
    for (int c = lane & 3; c < CH; c += 4) {
#pragma unroll
        for (int k = 0; k < LM_KT / 8; ++k)
            cp_async16(dst + ((lane >> 2) + 8 * k) * ST + c * 8, src[k] ? src[k] + c * 8 : pages, src[k] != nullptr);
    }
}

// One tile of LM_KT cached rows at `kt` (its first key is `key0`; keys from `khi` on are not seen) against the warp's 16
// query rows at `sq`: the scores, the online softmax (base 2) and O += P V for the warp's `cols` output columns from
// column `col0` of the rows.  Every tile a warp is given holds at least one key it sees.
template <int LM_COLS>
__device__ __forceinline__ void lm_tile(float (&o)[LM_COLS / 8][4], float& m0, float& m1, float& l0, float& l1, const bf16* sq,
                                        const bf16* kt, int ST, int W, int key0, int khi, int col0, int cols, float scale_log2,
                                        int lane) {
    const int tq = lane & 3;
    const int a_row = (((lane >> 3) & 1) << 3) + (lane & 7), a_dof = (lane >> 4) << 3;
    const int b_key = ((lane >> 4) << 3) + (lane & 7), b_dof = ((lane >> 3) & 1) << 3;
    const int v_key = (((lane >> 3) & 1) << 3) + (lane & 7), v_dof = (lane >> 4) << 3;
    float sc[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
    for (int ks = 0; ks < W / 16; ++ks) {
        uint32_t a[4], b0[4], b1[4];
        ldmatrix_x4(a, sq + a_row * ST + ks * 16 + a_dof);
        ldmatrix_x4(b0, kt + b_key * ST + ks * 16 + b_dof);
        ldmatrix_x4(b1, kt + (16 + b_key) * ST + ks * 16 + b_dof);
        mma_bf16(sc[0], a, b0[0], b0[1]);
        mma_bf16(sc[1], a, b0[2], b0[3]);
        mma_bf16(sc[2], a, b1[0], b1[1]);
        mma_bf16(sc[3], a, b1[2], b1[3]);
    }
    if (key0 + LM_KT > khi) {                                // the last tile: keys from khi on do not exist (or are not visible)
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e)
                if (key0 + n * 8 + 2 * tq + e >= khi) sc[n][e] = sc[n][2 + e] = -INFINITY;
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 4; ++n) {
        mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
        mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);          // finite: every tile holds a visible key
    const float u0 = n0 * scale_log2, u1 = n1 * scale_log2;
    const float c0 = fast_exp2(m0 * scale_log2 - u0), c1 = fast_exp2(m1 * scale_log2 - u1);
    m0 = n0;
    m1 = n1;
    l0 *= c0;
    l1 *= c1;
#pragma unroll
    for (int j = 0; j < LM_COLS / 8; ++j) {
        o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1;
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
        sc[n][0] = fast_exp2(sc[n][0] * scale_log2 - u0);
        sc[n][1] = fast_exp2(sc[n][1] * scale_log2 - u0);
        sc[n][2] = fast_exp2(sc[n][2] * scale_log2 - u1);
        sc[n][3] = fast_exp2(sc[n][3] * scale_log2 - u1);
        l0 += sc[n][0] + sc[n][1];
        l1 += sc[n][2] + sc[n][3];
    }
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
        uint32_t pf[4];
        pf[0] = pack_bf16(sc[2 * kb][0], sc[2 * kb][1]);
        pf[1] = pack_bf16(sc[2 * kb][2], sc[2 * kb][3]);
        pf[2] = pack_bf16(sc[2 * kb + 1][0], sc[2 * kb + 1][1]);
        pf[3] = pack_bf16(sc[2 * kb + 1][2], sc[2 * kb + 1][3]);
        const bf16* vrows = kt + (size_t)kb * 16 * ST + col0;
#pragma unroll
        for (int dp = 0; dp < LM_COLS / 16; ++dp) {
            if (dp * 16 < cols) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vrows + v_key * ST + dp * 16 + v_dof);
                mma_bf16(o[2 * dp], pf, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pf, b[2], b[3]);
            }
        }
    }
}

// The factors that turn a row's unnormalised sums into its output when the denominator also holds 2^(sink log2 e): with
// M the row's maximum (base 2, scaled) and Mn = max(M, sink'), out = O 2^(M - Mn) / (l 2^(M - Mn) + 2^(sink' - Mn)).
__device__ __forceinline__ void lm_sink(float& inv0, float& inv1, float l0, float l1, float M0, float M1,
                                        const float* __restrict__ sink, int ha, int hb, int H) {
    const float s0 = (ha < H ? sink[ha] : 0.f) * 1.4426950408889634f, s1 = (hb < H ? sink[hb] : 0.f) * 1.4426950408889634f;
    const float n0 = fmaxf(M0, s0), n1 = fmaxf(M1, s1);
    const float c0 = fast_exp2(M0 - n0), c1 = fast_exp2(M1 - n1);
    inv0 = c0 / (l0 * c0 + fast_exp2(s0 - n0));
    inv1 = c1 / (l1 * c1 + fast_exp2(s1 - n1));
}

template <int LM_COLS>       // output columns per warp: 128 or 256
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q_lat,
    const bf16* __restrict__ q_rot, const bf16* __restrict__ pages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ positions, const int* __restrict__ seq_idx, int page_size, int N, int H, int R, int Dr,
    float scale_log2, int split_keys, int n_splits, int warps_per_block, int num_pages, int* __restrict__ status,
    const float* __restrict__ sink) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int W = R + Dr, ST = W + 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int HG = (H + 15) / 16, RCH = (R + LM_COLS - 1) / LM_COLS;
    pdl_trigger();
    pdl_wait();
    long long w = (long long)blockIdx.x * warps_per_block + warp;
    if (warp >= warps_per_block || w >= (long long)N * HG * RCH * n_splits) return;
    const int split = (int)(w % n_splits);
    w /= n_splits;
    const int rc = (int)(w % RCH);
    w /= RCH;
    const int hg = (int)(w % HG);
    const int t = (int)(w / HG);
    bf16* sq = reinterpret_cast<bf16*>(lm_smem) + (size_t)warp * (16 + 2 * LM_KT) * ST;     // [16][ST] queries
    bf16* sk = sq + 16 * ST;                                                                // 2 x [LM_KT][ST] cached rows
    const int h0 = hg * 16, col0 = rc * LM_COLS;
    const int g = lane >> 2, tq = lane & 3;
    const int kend = positions[t] + 1;
    const int kbeg = split * split_keys, khi = min(kend, kbeg + split_keys);
    if (kbeg >= khi) {                                       // this range holds no key of the row
        if (rc == 0 && tq == 0) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = h0 + g + 8 * e;
                if (h < H) {
                    float* ml = part_ml + (((size_t)t * H + h) * n_splits + split) * 2;
                    ml[0] = -INFINITY;
                    ml[1] = 0.f;
                }
            }
        }
        return;
    }
    const ZaiTableRow table{block_table + (size_t)seq_idx[t] * table_width, table_width, num_pages, status};
    // the 16 heads' queries [latent part | rotated part]; heads beyond H are zeros
    for (int idx = lane; idx < 16 * (W / 8); idx += 32) {
        const int r = idx / (W / 8), c = (idx - r * (W / 8)) * 8;
        const bool valid = h0 + r < H;
        const size_t th = (size_t)t * H + (valid ? h0 + r : 0);
        const bf16* src = c < R ? q_lat + th * R + c : q_rot + th * Dr + (c - R);
        cp_async16(sq + r * ST + c, src, valid);
    }
    lm_load_tile(sk, ST, pages, table, kbeg, khi, page_size, W, lane);
    cp_async_commit();
    float o[LM_COLS / 8][4];
#pragma unroll
    for (int i = 0; i < LM_COLS / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;          // heads g and g+8 of the warp's 16
    const int n_tiles = (khi - kbeg + LM_KT - 1) / LM_KT;
    const int cols = min(LM_COLS, R - col0);                           // output columns of this warp (a multiple of 32)
    for (int i = 0; i < n_tiles; ++i) {
        const bf16* kt = sk + (size_t)(i & 1) * LM_KT * ST;
        if (i + 1 < n_tiles) {
            lm_load_tile(sk + (size_t)((i + 1) & 1) * LM_KT * ST, ST, pages, table, kbeg + (i + 1) * LM_KT, khi, page_size, W, lane);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        lm_tile<LM_COLS>(o, m0, m1, l0, l1, sq, kt, ST, W, kbeg + i * LM_KT, khi, col0, cols, scale_log2, lane);
        __syncwarp();                                        // the buffer is loaded again two tiles on
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int ha = h0 + g, hb = ha + 8;
    if (n_splits == 1) {
        float inv0 = 1.f / l0, inv1 = 1.f / l1;
        if (sink) lm_sink(inv0, inv1, l0, l1, m0 * scale_log2, m1 * scale_log2, sink, ha, hb, H);
#pragma unroll
        for (int j = 0; j < LM_COLS / 8; ++j) {
            const int d = j * 8 + 2 * tq;
            if (d < cols) {
                if (ha < H) *reinterpret_cast<uint32_t*>(out + ((size_t)t * H + ha) * R + col0 + d) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
                if (hb < H) *reinterpret_cast<uint32_t*>(out + ((size_t)t * H + hb) * R + col0 + d) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < LM_COLS / 8; ++j) {
        const int d = j * 8 + 2 * tq;
        if (d < cols) {
            if (ha < H) *reinterpret_cast<float2*>(part_o + (((size_t)t * H + ha) * n_splits + split) * R + col0 + d) = make_float2(o[j][0], o[j][1]);
            if (hb < H) *reinterpret_cast<float2*>(part_o + (((size_t)t * H + hb) * n_splits + split) * R + col0 + d) = make_float2(o[j][2], o[j][3]);
        }
    }
    if (rc == 0 && tq == 0) {
        if (ha < H) {
            float* ml = part_ml + (((size_t)t * H + ha) * n_splits + split) * 2;
            ml[0] = m0 * scale_log2;
            ml[1] = l0;
        }
        if (hb < H) {
            float* ml = part_ml + (((size_t)t * H + hb) * n_splits + split) * 2;
            ml[0] = m1 * scale_log2;
            ml[1] = l1;
        }
    }
}

// Steps of many rows: the four warps of a block share the tiles of cached rows.  A warp still owns one row of the step,
// 16 heads and a block of output columns; warps whose rows belong to one request form a group (in a long portion: all
// four, consecutive rows or the same row's other heads and columns), the whole block copies the group's tiles into one
// pair of buffers, and each member works on the tiles that hold keys it sees.  Groups of a block (at the border between two
// requests, or single tokens of several requests) take their turns one after the other.
template <int LM_COLS>
__global__ void __launch_bounds__(128) latent_attention_rows_kernel(
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ q_lat,
    const bf16* __restrict__ q_rot, const bf16* __restrict__ pages, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ positions, const int* __restrict__ seq_idx, int page_size, int N, int H, int R, int Dr,
    float scale_log2, int split_keys, int n_splits, int num_pages, int* __restrict__ status, const float* __restrict__ sink) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    __shared__ int s_key[4], s_khi[4];
    const int W = R + Dr, ST = W + 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int HG = (H + 15) / 16, RCH = (R + LM_COLS - 1) / LM_COLS;
    pdl_trigger();
    pdl_wait();
    // groups of heads fastest, then blocks of columns, then ranges of keys, then rows: neighbours share their cached rows
    long long w = (long long)blockIdx.x * 4 + warp;
    const bool live = w < (long long)N * n_splits * RCH * HG;
    const int hg = live ? (int)(w % HG) : 0;
    w /= HG;
    const int rc = live ? (int)(w % RCH) : 0;
    w /= RCH;
    const int split = live ? (int)(w % n_splits) : 0;
    const int t = live ? (int)(w / n_splits) : 0;
    bf16* sq = reinterpret_cast<bf16*>(lm_smem) + (size_t)warp * 16 * ST;         // [16][ST] this warp's queries
    bf16* sk = reinterpret_cast<bf16*>(lm_smem) + (size_t)4 * 16 * ST;            // 2 x [LM_KT][ST] the block's cached rows
    const int h0 = hg * 16, col0 = rc * LM_COLS;
    const int g = lane >> 2, tq = lane & 3;
    const int my_kbeg = split * split_keys;
    const int my_khi = live ? min(positions[t] + 1, my_kbeg + split_keys) : 0;
    const bool empty = !live || my_kbeg >= my_khi;           // (a range that holds no key of the row)
    const int my_key = empty ? -1 : seq_idx[t] * n_splits + split;               // what a group shares: the request and the range
    if (lane == 0) {
        s_key[warp] = my_key;
        s_khi[warp] = my_khi;
    }
    if (!empty) {
        for (int idx = lane; idx < 16 * (W / 8); idx += 32) {
            const int r = idx / (W / 8), c = (idx - r * (W / 8)) * 8;
            const bool valid = h0 + r < H;
            const size_t th = (size_t)t * H + (valid ? h0 + r : 0);
            const bf16* src = c < R ? q_lat + th * R + c : q_rot + th * Dr + (c - R);
            cp_async16(sq + r * ST + c, src, valid);
        }
    }
    cp_async_commit();
    float o[LM_COLS / 8][4];
#pragma unroll
    for (int i = 0; i < LM_COLS / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int cols = min(LM_COLS, R - col0);
    __syncthreads();
    for (int leader = 0; leader < 4; ++leader) {
        const int key = s_key[leader];
        bool first = key >= 0;                               // (the same for every thread: all read shared memory)
        for (int e = 0; e < leader; ++e) first = first && s_key[e] != key;
        if (!first) continue;
        int kmax = 0;
        for (int e = leader; e < 4; ++e)
            if (s_key[e] == key) kmax = max(kmax, s_khi[e]);
        const bool member = my_key == key;
        const int kbeg = (key % n_splits) * split_keys;
        const ZaiTableRow table{block_table + (size_t)(key / n_splits) * table_width, table_width, num_pages, status};
        const int n_tiles = (kmax - kbeg + LM_KT - 1) / LM_KT;
        // a tile: row tid / 4 of the 32, sixteen bytes a copy, four threads a row
        auto load = [&](int i) {
            const int j = kbeg + i * LM_KT + (tid >> 2);
            const bf16* src = j < kmax ? pages + ((size_t)table.page(j / page_size) * page_size + j % page_size) * W : nullptr;
            bf16* dst = sk + (size_t)(i & 1) * LM_KT * ST + (tid >> 2) * ST;
            for (int c = tid & 3; c < W / 8; c += 4) cp_async16(dst + c * 8, src ? src + c * 8 : pages, src != nullptr);
        };
        load(0);
        cp_async_commit();
        for (int i = 0; i < n_tiles; ++i) {
            if (i + 1 < n_tiles) {
                load(i + 1);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            if (member && kbeg + i * LM_KT < my_khi)
                lm_tile<LM_COLS>(o, m0, m1, l0, l1, sq, sk + (size_t)(i & 1) * LM_KT * ST, ST, W, kbeg + i * LM_KT, my_khi, col0, cols,
                                 scale_log2, lane);
            __syncthreads();                                 // the buffer is loaded again two tiles on
        }
    }
    if (!live) return;
    const int ha = h0 + g, hb = ha + 8;
    if (empty) {                                             // (only with several ranges)
        if (rc == 0 && tq == 0) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int h = e ? hb : ha;
                if (h < H) {
                    float* ml = part_ml + (((size_t)t * H + h) * n_splits + split) * 2;
                    ml[0] = -INFINITY;
                    ml[1] = 0.f;
                }
            }
        }
        return;
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (n_splits == 1) {
        float inv0 = 1.f / l0, inv1 = 1.f / l1;
        if (sink) lm_sink(inv0, inv1, l0, l1, m0 * scale_log2, m1 * scale_log2, sink, ha, hb, H);
#pragma unroll
        for (int j = 0; j < LM_COLS / 8; ++j) {
            const int d = j * 8 + 2 * tq;
            if (d < cols) {
                if (ha < H) *reinterpret_cast<uint32_t*>(out + ((size_t)t * H + ha) * R + col0 + d) = pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
                if (hb < H) *reinterpret_cast<uint32_t*>(out + ((size_t)t * H + hb) * R + col0 + d) = pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < LM_COLS / 8; ++j) {
        const int d = j * 8 + 2 * tq;
        if (d < cols) {
            if (ha < H) *reinterpret_cast<float2*>(part_o + (((size_t)t * H + ha) * n_splits + split) * R + col0 + d) = make_float2(o[j][0], o[j][1]);
            if (hb < H) *reinterpret_cast<float2*>(part_o + (((size_t)t * H + hb) * n_splits + split) * R + col0 + d) = make_float2(o[j][2], o[j][3]);
        }
    }
    if (rc == 0 && tq == 0) {
        if (ha < H) {
            float* ml = part_ml + (((size_t)t * H + ha) * n_splits + split) * 2;
            ml[0] = m0 * scale_log2;
            ml[1] = l0;
        }
        if (hb < H) {
            float* ml = part_ml + (((size_t)t * H + hb) * n_splits + split) * 2;
            ml[0] = m1 * scale_log2;
            ml[1] = l1;
        }
    }
}

// out[t, h, :] = sum_c O_c 2^(m_c - m) / sum_c l_c 2^(m_c - m), the ranges taken in order
__global__ void latent_combine_kernel(bf16* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      int R, int n_splits, int H, const float* __restrict__ sink) {
    pdl_trigger();
    pdl_wait();
    const size_t th = blockIdx.x;
    const float* ml = part_ml + th * n_splits * 2;
    const float sk = sink ? sink[th % H] * 1.4426950408889634f : -INFINITY;
    float m = sk;
    for (int c = 0; c < n_splits; ++c) m = fmaxf(m, ml[2 * c]);
    float l = sink ? fast_exp2(sk - m) : 0.f;
    for (int c = 0; c < n_splits; ++c) l += ml[2 * c + 1] * fast_exp2(ml[2 * c] - m);
    const float inv = 1.f / l;
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < n_splits; ++c) {
            const float wgt = fast_exp2(ml[2 * c] - m);              // an empty range: 2^-inf = 0, its O is never read
            if (wgt > 0.f) acc += part_o[(th * n_splits + c) * R + d] * wgt;
        }
        out[th * R + d] = __float2bfloat16_rn(acc * inv);
    }
}

ZAI_API int zai_latent_attention_mma_supports(int R, int Dr) {
    const int W = R + Dr;
    return R >= 32 && R % 32 == 0 && Dr >= 0 && W % 16 == 0 && (size_t)(4 * 16 + 2 * LM_KT) * (W + 8) * 2 <= 200 * 1024;
}

// bfloat16; part_o [N, H, n_splits, R] and part_ml [N, H, n_splits, 2] 32-bit scratch (unused with n_splits = 1).
ZAI_API int zai_latent_attention_mma(void* out, float* part_o, float* part_ml, const void* q_lat, const void* q_rot, const void* pages,
                                     const int* block_table, int table_width, const int* positions, const int* seq_idx,
                                     int page_size, int N, int H, int R, int Dr, float scale, int split_keys, int n_splits,
                                     int num_pages, int* status, const float* sink, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (!zai_latent_attention_mma_supports(R, Dr) || H < 1 || n_splits < 1 || split_keys < LM_KT || split_keys % LM_KT) return ZAI_BAD_SIZE;
    const int cols = R <= 128 ? 128 : 256;
    const int sharers = ((H + 15) / 16) * ((R + cols - 1) / cols);      // warps that read the same cached rows
    if (n_splits == 1 || (sharers >= 2 && (long long)N * sharers * n_splits >= 1024)) {
        // many rows, or several groups of heads (blocks of columns) a row and warps enough to fill the device although a
        // block's groups take turns: four warps a block share the tiles
        const size_t smem = (size_t)(4 * 16 + 2 * LM_KT) * (R + Dr + 8) * 2;
        const long long warps = (long long)N * sharers * n_splits;
        const long long blocks = (warps + 3) / 4;
        if (blocks > 0x7fffffffLL || smem > 200 * 1024) return ZAI_BAD_SIZE;
        static unsigned long long done_rows = 0;
        if (zai_first_on_device(&done_rows)) {
            cudaFuncSetAttribute(latent_attention_rows_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            cudaFuncSetAttribute(latent_attention_rows_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        }
        auto rows_kernel = cols == 128 ? latent_attention_rows_kernel<128> : latent_attention_rows_kernel<256>;
        int rc = launch_pdl(rows_kernel, dim3((unsigned)blocks), dim3(128), smem, stream, (bf16*)out, part_o, part_ml,
                            (const bf16*)q_lat, (const bf16*)q_rot, (const bf16*)pages, block_table, table_width, positions, seq_idx,
                            page_size, N, H, R, Dr, scale * 1.4426950408889634f, split_keys, n_splits, num_pages, status, sink);
        if (rc != 0 || n_splits == 1) return rc;
        return launch_pdl(latent_combine_kernel, dim3((unsigned)((size_t)N * H)), dim3(128), 0, stream, (bf16*)out,
                          (const float*)part_o, (const float*)part_ml, R, n_splits, H, sink);
    }
    const size_t per_warp = (size_t)(16 + 2 * LM_KT) * (R + Dr + 8) * 2;
    int wpb = (int)((200 * 1024) / per_warp);
    wpb = wpb > 4 ? 4 : wpb;
    const long long warps = (long long)N * ((H + 15) / 16) * ((R + cols - 1) / cols) * n_splits;
    const long long blocks = (warps + wpb - 1) / wpb;
    if (blocks > 0x7fffffffLL) return ZAI_BAD_SIZE;
    static unsigned long long done = 0;
    if (zai_first_on_device(&done)) {
        cudaFuncSetAttribute(latent_attention_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(latent_attention_mma_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    auto kernel = cols == 128 ? latent_attention_mma_kernel<128> : latent_attention_mma_kernel<256>;
    int rc = launch_pdl(kernel, dim3((unsigned)blocks), dim3(128), per_warp * wpb, stream, (bf16*)out, part_o,
                        part_ml, (const bf16*)q_lat, (const bf16*)q_rot, (const bf16*)pages, block_table, table_width, positions,
                        seq_idx, page_size, N, H, R, Dr, scale * 1.4426950408889634f, split_keys, n_splits, wpb, num_pages, status, sink);
    if (rc != 0 || n_splits == 1) return rc;
    return launch_pdl(latent_combine_kernel, dim3((unsigned)((size_t)N * H)), dim3(128), 0, stream, (bf16*)out, (const float*)part_o,
                      (const float*)part_ml, R, n_splits, H, sink);
}

// out [N, H, R], q_lat [N, H, R], q_rot [N, H, Dr], pages [num_pages, page_size, R + Dr], all in `dtype`; sink [H] 32-bit or null.
ZAI_API int zai_latent_attention(void* out, const void* q_lat, const void* q_rot, const void* pages, int dtype, const int* block_table,
                                 int table_width, const int* positions, const int* seq_idx, int page_size, int N, int H, int R,
                                 int Dr, float scale, int num_pages, int* status, const float* sink, cudaStream_t stream) {
    if (N <= 0) return ZAI_OK;
    if (H < 1 || R < 1 || R > 1024 || Dr < 0 || H > 65535 * LA_WARPS) return ZAI_BAD_SIZE;
    if (((size_t)LA_WARPS * (R + Dr) + (size_t)LA_KEYS * (R + Dr + 1)) * sizeof(float) > 200 * 1024) return ZAI_BAD_SIZE;
#define LA_GO(MAXR)                                                                                                            \
    ZAI_DISPATCH(dtype, return (launch_latent<T, MAXR>(out, q_lat, q_rot, pages, block_table, table_width, positions, seq_idx, \
                                                       page_size, N, H, R, Dr, scale, num_pages, status, sink, stream)))
    if (R <= 128) LA_GO(4);
    else if (R <= 256) LA_GO(8);
    else if (R <= 512) LA_GO(16);
    else LA_GO(32);
#undef LA_GO
    return launch_status();
}
