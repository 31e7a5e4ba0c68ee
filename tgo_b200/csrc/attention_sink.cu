// Paged causal attention on the tensor cores for bfloat16 storage, of the kind that has keys
// and values of different widths, a sliding window and a sink:
//
//   score(i, j) = (q_i . k_j) * scale                 for max(0, i - window + 1) <= j <= i
//   w(i, j)     = exp(score(i, j)) / (exp(sink_h) + sum_j' exp(score(i, j')))
//   out_i       = sum_j w(i, j) v_j
//
// (window 0: every earlier key; sinks null: no sink.) With a soft cap c > 0 the scaled score
// goes through c tanh(score / c) first. A value row lies `v_row` elements after the one before
// it: dv for a plane of values, the key rows' width when a value is the first dv channels of
// its key row (one cache plane that serves as both). One CTA takes a tile of query rows of
// one request and one kv head: the rows are the (token, query head of the group) pairs of up
// to 128/G consecutive tokens, G = H/Hkv, so every row of the tile reads the same keys and
// values. Keys [page][kv head][offset][dk] and values [page][kv head][offset][dv] come through
// the request's block table, 64 at a time, by cp.async into shared memory (two buffers: the
// next tile loads while this one is computed), each row padded with zeros to the kernel's
// compile-time widths DK and DV. S = Q K^T and O += P V are mma.sync m16n8k16 with float32
// accumulators; the running maximum, the sum of exponentials, the sink and the rescaling are
// float32 in registers. Tiles are given by arrays (first token, token count) or, when those
// are null, tile t is the single token t (a step of single tokens). Such a step may cut each
// token's keys into `n_splits` ranges of key tiles, one CTA each: the partial results
// (unnormalised O, maximum, sum) go to scratch and `attention_sink_join_kernel` joins them and
// adds the sink.
// `keep_first` > 0 (with a window): the first keep_first keys of a request stay visible to
// every later query beside the window; the key tiles that hold them and lie before the
// window's first tile are walked first, then the window's tiles (one list of tiles, which is
// also what `n_splits` cuts). `dist_bias` (float32 [n_dist][H]): dist_bias[min(i - j, n_dist
// - 1)][h] is added to the scaled score, unscaled (a learned bias by distance).
#include "common.cuh"

#define AS_BN 64                 // keys per tile
#define AS_PAD 8                 // bf16 of padding per shared-memory row (keeps ldmatrix conflict-free)

#include "mma_sync.cuh"

#define AS_WARPS 4
#define AS_RW 2                  // m16 row tiles per warp
#define AS_BM (16 * AS_WARPS * AS_RW)
#define AS_LOG2E 1.4426950408889634f
#define AS_PAGES 320             // block-table entries of a CTA's key range kept in shared memory

// A raw product q . k as the softmax's exponent in base 2: scaled, and with a soft cap c
// (cap_log2 = c log2 e > 0, scale_over_cap = scale / c) bounded by c tanh(scale (q . k) / c).
// tanh(x) = 1 - 2 / (1 + e^(2x)) with the hardware's exponential and reciprocal, five
// instructions a score: C tanh(x) = C - 2C / (1 + 2^(2 log2(e) x)); an exponential that
// overflows gives a reciprocal of 0 and the bound C itself. Absolute error about 1e-7 C (the
// library's tanhf, many instructions and branches, cost more than the products).
__device__ __forceinline__ float as_scored(float qk, float scale_log2, float cap_log2, float scale_over_cap) {
    if (!(cap_log2 > 0.f)) return qk * scale_log2;
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(qk * (scale_over_cap * (2.f * AS_LOG2E))));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
    return fmaf(-2.f * cap_log2, r, cap_log2);
}

template <int DK, int DV>
__global__ void __launch_bounds__(AS_WARPS * 32)
attention_sink_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                      long long out_stride, const bf16* __restrict__ k_cache,
                      const bf16* __restrict__ v_cache, int page_size,
                      const int* __restrict__ block_tables, int max_blocks,
                      const int* __restrict__ positions, const int* __restrict__ seq_ids,
                      const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok, int H,
                      int Hkv, int dk, int dv, float scale_log2, int window,
                      const float* __restrict__ sinks, int n_splits, float* __restrict__ part_o,
                      float* __restrict__ part_ml, float cap_log2, float scale_over_cap, int v_row,
                      int keep_first, const float* __restrict__ dist_bias, int n_dist) {
    constexpr int LDK = DK + AS_PAD, LDV = DV + AS_PAD;
    constexpr int KS = DK / 16;
    constexpr int CHK = DK / 8, CHV = DV / 8;  // 16-byte chunks per padded row
    constexpr int THREADS = AS_WARPS * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                // [AS_BM][LDK]
    bf16* sk = sq + AS_BM * LDK;               // [2][AS_BN][LDK]
    bf16* sv = sk + 2 * AS_BN * LDK;           // [2][AS_BN][LDV]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // later tiles of a request read more keys: they are started first
    const int tile = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y;
    const int G = H / Hkv;
    const int tok0 = tile_tok0 ? tile_tok0[tile] : tile, ntok = tile_ntok ? tile_ntok[tile] : 1;
    const int n_rows = ntok * G;
    const int p0 = positions[tok0];            // position of the tile's first token
    if (p0 < 0) {                              // a request that brings nothing: zeros out
        for (int i = tid; i < n_rows * dv; i += THREADS) {
            const int r = i / dv, d = i % dv;
            out[(size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * dv + d] =
                __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok0] * max_blocks;
    const int p_last = p0 + ntok - 1;
    // keys any row of the tile may read: [key_lo, key_hi)
    const int key_lo = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int key_hi = p_last + 1;
    const int t_first = key_lo / AS_BN;        // the window's first tile
    // tiles of kept first keys that lie before it; the walk is over v = 0 .. n_kept - 1 (those
    // tiles), then the window's tiles: tile_of(v)
    int n_kept = keep_first > 0 ? (keep_first + AS_BN - 1) / AS_BN : 0;
    if (n_kept > t_first) n_kept = t_first;
    int t_lo = 0, t_hi = n_kept + (key_hi + AS_BN - 1) / AS_BN - t_first;
    if (n_splits > 1) {                        // this CTA's share of the key tiles (it may be empty)
        const int per = (t_hi - t_lo + n_splits - 1) / n_splits;
        t_lo += blockIdx.z * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }
    auto tile_of = [&](int v) { return v < n_kept ? v : t_first + (v - n_kept); };
    const int chk = dk / 8, chv = dv / 8;      // chunks a real row has

    for (int i = tid; i < AS_BM * CHK; i += THREADS) {
        const int r = i / CHK, c = i % CHK;
        const bool ok = r < n_rows && c < chk;
        const bf16* src = ok ? q + (size_t)(tok0 + r / G) * q_stride + (size_t)(kvh * G + r % G) * dk + c * 8 : q;
        cp_async16(sq + r * LDK + c * 8, src, ok);
    }
    auto load_kv = [&](int t, int buf) {
        bf16* dks = sk + buf * AS_BN * LDK;
        bf16* dvs = sv + buf * AS_BN * LDV;
        for (int i = tid; i < AS_BN * CHK; i += THREADS) {
            const int r = i / CHK, c = i % CHK;
            const int j = t * AS_BN + r;
            const bool ok = (j >= key_lo || j < keep_first) && j < key_hi && c < chk;
            size_t off = 0;
            if (ok) {
                const int pi = j / page_size, po = j - pi * page_size;
                off = (((size_t)bt[pi] * Hkv + kvh) * page_size + po) * dk + c * 8;
            }
            cp_async16(dks + r * LDK + c * 8, k_cache + off, ok);
        }
        for (int i = tid; i < AS_BN * CHV; i += THREADS) {
            const int r = i / CHV, c = i % CHV;
            const int j = t * AS_BN + r;
            const bool ok = (j >= key_lo || j < keep_first) && j < key_hi && c < chv;
            size_t off = 0;
            if (ok) {
                const int pi = j / page_size, po = j - pi * page_size;
                off = (((size_t)bt[pi] * Hkv + kvh) * page_size + po) * v_row + c * 8;
            }
            cp_async16(dvs + r * LDV + c * 8, v_cache + off, ok);
        }
    };
    if (t_lo < t_hi) load_kv(tile_of(t_lo), 0);
    cp_async_commit();

    float o[AS_RW][DV / 8][4];
    float m_run[AS_RW][2], l_run[AS_RW][2];
    int pos_row[AS_RW][2], vis_row[AS_RW][2];
    const float* bias_row[AS_RW][2];           // the distance bias's column of each row's head
#pragma unroll
    for (int rw = 0; rw < AS_RW; ++rw) {
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) { o[rw][i][0] = o[rw][i][1] = o[rw][i][2] = o[rw][i][3] = 0.f; }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (warp * AS_RW + rw) * 16 + (lane >> 2) + 8 * h;
            m_run[rw][h] = -INFINITY;
            l_run[rw][h] = 0.f;
            pos_row[rw][h] = r < n_rows ? p0 + r / G : -1;      // rows beyond the tile read nothing
            vis_row[rw][h] = (window > 0 && pos_row[rw][h] - window + 1 > 0) ? pos_row[rw][h] - window + 1 : 0;
            bias_row[rw][h] = dist_bias ? dist_bias + kvh * G + (r < n_rows ? r % G : 0) : nullptr;
        }
    }
    const bool warp_active = warp * AS_RW * 16 < n_rows;
    // a scaled (and capped) score with the bias of its distance, as an exponent in base 2
    auto biased = [&](float sc, const float* col, int dist) {
        return col ? fmaf(col[(size_t)(dist < n_dist ? dist : n_dist - 1) * H], AS_LOG2E, sc) : sc;
    };

    for (int vt_i = t_lo; vt_i < t_hi; ++vt_i) {
        const int t = tile_of(vt_i);
        const int buf = (vt_i - t_lo) & 1;
        if (vt_i + 1 < t_hi) load_kv(tile_of(vt_i + 1), buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (warp_active) {
            const bf16* kt = sk + buf * AS_BN * LDK;
            const bf16* vt = sv + buf * AS_BN * LDV;
            float s[AS_RW][AS_BN / 8][4];
#pragma unroll
            for (int rw = 0; rw < AS_RW; ++rw)
#pragma unroll
                for (int i = 0; i < AS_BN / 8; ++i) { s[rw][i][0] = s[rw][i][1] = s[rw][i][2] = s[rw][i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t qa[AS_RW][4];
#pragma unroll
                for (int rw = 0; rw < AS_RW; ++rw)
                    ldmatrix_x4(qa[rw], sq + ((warp * AS_RW + rw) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK +
                                            ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < AS_BN / 16; ++np) {       // two n-tiles (16 keys) at a time
                    uint32_t kb[4];
                    ldmatrix_x4(kb, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + ks * 16 +
                                        ((lane >> 3) & 1) * 8);
#pragma unroll
                    for (int rw = 0; rw < AS_RW; ++rw) {
                        mma_bf16(s[rw][2 * np], qa[rw], kb[0], kb[1]);
                        mma_bf16(s[rw][2 * np + 1], qa[rw], kb[2], kb[3]);
                    }
                }
            }
            // a tile that lies wholly inside every row's range needs no mask
            const int first_row_pos = p0 + (warp * AS_RW * 16) / G;
            const bool full = (t + 1) * AS_BN - 1 <= first_row_pos && t * AS_BN >= key_lo &&
                              (window == 0 || t * AS_BN >= p_last - window + 1) &&
                              (warp * AS_RW + AS_RW) * 16 <= n_rows;
            const int kbase = t * AS_BN + (lane & 3) * 2;
            uint32_t pa[AS_RW][AS_BN / 16][4];
#pragma unroll
            for (int rw = 0; rw < AS_RW; ++rw) {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < AS_BN / 8; ++i) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = kbase + i * 8 + e;
                        const bool a = full || (j <= pos_row[rw][0] && (j >= vis_row[rw][0] || j < keep_first));
                        const bool c = full || (j <= pos_row[rw][1] && (j >= vis_row[rw][1] || j < keep_first));
                        s[rw][i][e] = a ? biased(as_scored(s[rw][i][e], scale_log2, cap_log2, scale_over_cap),
                                                 bias_row[rw][0], pos_row[rw][0] - j) : -INFINITY;
                        s[rw][i][2 + e] = c ? biased(as_scored(s[rw][i][2 + e], scale_log2, cap_log2, scale_over_cap),
                                                     bias_row[rw][1], pos_row[rw][1] - j) : -INFINITY;
                        mx[0] = fmaxf(mx[0], s[rw][i][e]);
                        mx[1] = fmaxf(mx[1], s[rw][i][2 + e]);
                    }
                }
                float corr[2], base[2], sum[2] = {0.f, 0.f};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                    const float mn = fmaxf(m_run[rw][h], mx[h]);
                    // a row that has seen no key yet keeps base 0 so that exp2(-inf - 0) = 0
                    base[h] = mn == -INFINITY ? 0.f : mn;
                    corr[h] = exp2f(m_run[rw][h] - base[h]);
                    m_run[rw][h] = mn;
                }
#pragma unroll
                for (int i = 0; i < AS_BN / 8; ++i) {
                    s[rw][i][0] = exp2f(s[rw][i][0] - base[0]);
                    s[rw][i][1] = exp2f(s[rw][i][1] - base[0]);
                    s[rw][i][2] = exp2f(s[rw][i][2] - base[1]);
                    s[rw][i][3] = exp2f(s[rw][i][3] - base[1]);
                    sum[0] += s[rw][i][0] + s[rw][i][1];
                    sum[1] += s[rw][i][2] + s[rw][i][3];
                }
                l_run[rw][0] = l_run[rw][0] * corr[0] + sum[0];     // per-lane partial sums
                l_run[rw][1] = l_run[rw][1] * corr[1] + sum[1];
#pragma unroll
                for (int i = 0; i < DV / 8; ++i) {
                    o[rw][i][0] *= corr[0]; o[rw][i][1] *= corr[0];
                    o[rw][i][2] *= corr[1]; o[rw][i][3] *= corr[1];
                }
#pragma unroll
                for (int kk = 0; kk < AS_BN / 16; ++kk) {
                    pa[rw][kk][0] = pack_bf16(s[rw][2 * kk][0], s[rw][2 * kk][1]);
                    pa[rw][kk][1] = pack_bf16(s[rw][2 * kk][2], s[rw][2 * kk][3]);
                    pa[rw][kk][2] = pack_bf16(s[rw][2 * kk + 1][0], s[rw][2 * kk + 1][1]);
                    pa[rw][kk][3] = pack_bf16(s[rw][2 * kk + 1][2], s[rw][2 * kk + 1][3]);
                }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < AS_BN / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < DV / 16; ++dp) {          // two n-tiles (16 dims) at a time
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV +
                                              dp * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int rw = 0; rw < AS_RW; ++rw) {
                        mma_bf16(o[rw][2 * dp], pa[rw][kk], vb[0], vb[1]);
                        mma_bf16(o[rw][2 * dp + 1], pa[rw][kk], vb[2], vb[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (!warp_active) return;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int rw = 0; rw < AS_RW; ++rw) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float l = l_run[rw][h];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const int r = (warp * AS_RW + rw) * 16 + (lane >> 2) + 8 * h;
            if (r >= n_rows) continue;
            const int head = kvh * G + r % G;
            if (n_splits > 1) {                // a share of the keys: the join kernel finishes
                const size_t at = ((size_t)(tok0 + r / G) * H + head) * n_splits + blockIdx.z;
                if ((lane & 3) == 0) {
                    part_ml[at * 2] = m_run[rw][h];
                    part_ml[at * 2 + 1] = l;
                }
                float* po = part_o + at * dv + col;
#pragma unroll
                for (int i = 0; i < DV / 8; ++i)
                    if (i * 8 + col < dv) *(float2*)(po + i * 8) = make_float2(o[rw][i][2 * h], o[rw][i][2 * h + 1]);
                continue;
            }
            float corr = 1.f;
            if (sinks) {                       // the sink joins the denominator last
                const float sk2 = sinks[head] * AS_LOG2E, m = m_run[rw][h];
                const float mn = fmaxf(m, sk2);
                corr = exp2f(m - mn);          // m = -inf cannot happen here: a row sees itself
                l = l * corr + exp2f(sk2 - mn);
            }
            const float inv = l > 0.f ? corr / l : 0.f;
            bf16* dst = out + (size_t)(tok0 + r / G) * out_stride + (size_t)head * dv + col;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i)
                if (i * 8 + col < dv)
                    *(uint32_t*)(dst + i * 8) = pack_bf16(o[rw][i][2 * h] * inv, o[rw][i][2 * h + 1] * inv);
        }
    }
}

// A step of single tokens with at most 16 query heads a kv head: the heads are the rows of one
// m16 tile, which all four warps hold; each 64-key tile is loaded by the whole CTA and warp w
// takes its keys 16w .. 16w+15, keeping its own maximum, sum and O. At the end the four
// partial states are joined through shared memory in warp order; the sink is added there, or,
// with n_splits > 1, the CTA's share goes to scratch for the join kernel.
template <int DK, int DV>
__global__ void __launch_bounds__(128)
attention_sink_decode_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                             long long out_stride, const bf16* __restrict__ k_cache,
                             const bf16* __restrict__ v_cache, int page_size,
                             const int* __restrict__ block_tables, int max_blocks,
                             const int* __restrict__ positions, const int* __restrict__ seq_ids, int H,
                             int Hkv, int dk, int dv, float scale_log2, int window,
                             const float* __restrict__ sinks, int n_splits, float* __restrict__ part_o,
                             float* __restrict__ part_ml, float cap_log2, float scale_over_cap, int v_row,
                             int keep_first, const float* __restrict__ dist_bias, int n_dist) {
    constexpr int LDK = DK + AS_PAD, LDV = DV + AS_PAD;
    constexpr int KS = DK / 16;
    constexpr int CHK = DK / 8, CHV = DV / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                // [16][LDK]
    bf16* sk = sq + 16 * LDK;                  // [2][64][LDK]
    bf16* sv = sk + 2 * AS_BN * LDK;           // [2][64][LDV]
    __shared__ float s_ml[4][16][2];
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = H / Hkv;
    const int p = positions[tok];
    if (p < 0) {                               // a request that brings nothing: zeros out
        if (split == 0)
            for (int i = tid; i < G * dv; i += 128)
                out[(size_t)tok * out_stride + (size_t)(kvh * G) * dv + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok] * max_blocks;
    const int key_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int key_hi = p + 1;
    const int t_first = key_lo / AS_BN;        // the window's first tile
    // tiles of kept first keys before it are walked first: v = 0 .. n_kept - 1, then the window's
    int n_kept = keep_first > 0 ? (keep_first + AS_BN - 1) / AS_BN : 0;
    if (n_kept > t_first) n_kept = t_first;
    int t_lo = 0, t_hi = n_kept + (key_hi + AS_BN - 1) / AS_BN - t_first;
    if (n_splits > 1) {
        const int per = (t_hi - t_lo + n_splits - 1) / n_splits;
        t_lo += split * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }
    auto tile_of = [&](int v) { return v < n_kept ? v : t_first + (v - n_kept); };
    const int chk = dk / 8, chv = dv / 8;
    // this CTA's slice of the block table (the window's part of its share) -> shared memory, so
    // that the address of a row is not a chain of two global loads
    __shared__ int s_pages[AS_PAGES];
    const int w_lo = t_lo > n_kept ? t_lo : n_kept;       // first walk index inside the window
    const int pg_lo = w_lo < t_hi ? (tile_of(w_lo) * AS_BN) / page_size : 0;
    int pg_hi = w_lo < t_hi ? (tile_of(t_hi - 1) * AS_BN + AS_BN + page_size - 1) / page_size : 0;
    if (pg_hi > max_blocks) pg_hi = max_blocks;
    if (pg_hi - pg_lo > AS_PAGES) pg_hi = pg_lo + AS_PAGES;
    for (int i = pg_lo + tid; i < pg_hi; i += 128) s_pages[i - pg_lo] = bt[i];
    __syncthreads();
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    auto page_of = [&](int pi) { return (pi >= pg_lo && pi < pg_hi) ? s_pages[pi - pg_lo] : bt[pi]; };
    for (int i = tid; i < 16 * CHK; i += 128) {
        const int r = i / CHK, c = i % CHK;
        const bool ok = r < G && c < chk;
        cp_async16(sq + r * LDK + c * 8,
                   ok ? q + (size_t)tok * q_stride + (size_t)(kvh * G + r) * dk + c * 8 : q, ok);
    }
    auto load_kv = [&](int t, int buf) {
        bf16* dks = sk + buf * AS_BN * LDK;
        bf16* dvs = sv + buf * AS_BN * LDV;
        for (int i = tid; i < AS_BN * CHK; i += 128) {
            const int r = i / CHK, c = i % CHK;
            const int j = t * AS_BN + r;
            const bool ok = (j >= key_lo || j < keep_first) && j < key_hi && c < chk;
            size_t off = 0;
            if (ok) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / page_size, po = j - pi * page_size;
                off = (((size_t)page_of(pi) * Hkv + kvh) * page_size + po) * dk + c * 8;
            }
            cp_async16(dks + r * LDK + c * 8, k_cache + off, ok);
        }
        for (int i = tid; i < AS_BN * CHV; i += 128) {
            const int r = i / CHV, c = i % CHV;
            const int j = t * AS_BN + r;
            const bool ok = (j >= key_lo || j < keep_first) && j < key_hi && c < chv;
            size_t off = 0;
            if (ok) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / page_size, po = j - pi * page_size;
                off = (((size_t)page_of(pi) * Hkv + kvh) * page_size + po) * v_row + c * 8;
            }
            cp_async16(dvs + r * LDV + c * 8, v_cache + off, ok);
        }
    };
    if (t_lo < t_hi) load_kv(tile_of(t_lo), 0);
    cp_async_commit();

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const bool row_lo_ok = r_lo < G, row_hi_ok = r_hi < G;
    uint32_t qa[KS][4];
    const float* bias_lo = dist_bias ? dist_bias + kvh * G + (row_lo_ok ? r_lo : 0) : nullptr;
    const float* bias_hi = dist_bias ? dist_bias + kvh * G + (row_hi_ok ? r_hi : 0) : nullptr;
    auto biased = [&](float sc, const float* col, int dist) {
        return col ? fmaf(col[(size_t)(dist < n_dist ? dist : n_dist - 1) * H], AS_LOG2E, sc) : sc;
    };

    for (int vt_i = t_lo; vt_i < t_hi; ++vt_i) {
        const int t = tile_of(vt_i);
        const int buf = (vt_i - t_lo) & 1;
        if (vt_i + 1 < t_hi) load_kv(tile_of(vt_i + 1), buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (vt_i == t_lo) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                ldmatrix_x4(qa[ks], sq + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDK + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* kt = sk + buf * AS_BN * LDK + warp * 16 * LDK;
        const bf16* vt = sv + buf * AS_BN * LDV + warp * 16 * LDV;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t kb[4];
            ldmatrix_x4(kb, kt + ((lane & 7) + (lane >> 4) * 8) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[0], qa[ks], kb[0], kb[1]);
            mma_bf16(s[1], qa[ks], kb[2], kb[3]);
        }
        const int kbase = t * AS_BN + warp * 16 + (lane & 3) * 2;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = kbase + i * 8 + e;
                const bool vis = (j >= key_lo || j < keep_first) && j < key_hi;
                s[i][e] = (vis && row_lo_ok) ? biased(as_scored(s[i][e], scale_log2, cap_log2, scale_over_cap),
                                                      bias_lo, p - j) : -INFINITY;
                s[i][2 + e] = (vis && row_hi_ok) ? biased(as_scored(s[i][2 + e], scale_log2, cap_log2, scale_over_cap),
                                                          bias_hi, p - j) : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[i][e]);
                mx_hi = fmaxf(mx_hi, s[i][2 + e]);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo;
        const float base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            s[i][0] = exp2f(s[i][0] - base_lo);
            s[i][1] = exp2f(s[i][1] - base_lo);
            s[i][2] = exp2f(s[i][2] - base_hi);
            s[i][3] = exp2f(s[i][3] - base_hi);
            sum_lo += s[i][0] + s[i][1];
            sum_hi += s[i][2] + s[i][3];
        }
        l_lo = l_lo * corr_lo + sum_lo;
        l_hi = l_hi * corr_hi + sum_hi;
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < DV / 16; ++dp) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDV + dp * 16 + (lane >> 4) * 8);
            o[2 * dp][0] *= corr_lo; o[2 * dp][1] *= corr_lo;
            o[2 * dp][2] *= corr_hi; o[2 * dp][3] *= corr_hi;
            o[2 * dp + 1][0] *= corr_lo; o[2 * dp + 1][1] *= corr_lo;
            o[2 * dp + 1][2] *= corr_hi; o[2 * dp + 1][3] *= corr_hi;
            mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
            mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();
    // join the four warps' states: O through the (now free) key buffers and, if they are too
    // small for it, the value buffers behind them ([4][16][DV] floats in all)
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    float* so = (float*)sk;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
        *(float2*)(so + ((size_t)warp * 16 + r_lo) * DV + i * 8 + col) = make_float2(o[i][0], o[i][1]);
        *(float2*)(so + ((size_t)warp * 16 + r_hi) * DV + i * 8 + col) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
        s_ml[warp][r_lo][0] = m_lo; s_ml[warp][r_lo][1] = l_lo;
        s_ml[warp][r_hi][0] = m_hi; s_ml[warp][r_hi][1] = l_hi;
    }
    __syncthreads();
    for (int i = tid; i < G * dv; i += 128) {
        const int r = i / dv, d = i % dv;
        const int head = kvh * G + r;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, s_ml[w][r][0]);
        const float sk2 = (sinks && n_splits == 1) ? sinks[head] * AS_LOG2E : -INFINITY;
        const float mj = fmaxf(m, sk2);
        float l = sk2 != -INFINITY ? exp2f(sk2 - mj) : 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = s_ml[w][r][0];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - mj);
                l += s_ml[w][r][1] * f;
                acc += so[((size_t)w * 16 + r) * DV + d] * f;
            }
        }
        if (n_splits > 1) {
            const size_t at = ((size_t)tok * H + head) * n_splits + split;
            part_o[at * dv + d] = acc;
            if (d == 0) {
                part_ml[at * 2] = m;
                part_ml[at * 2 + 1] = l;
            }
        } else {
            out[(size_t)tok * out_stride + (size_t)head * dv + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        }
    }
}

// Wide rows whose values are the first dv channels of the key rows (one cache plane, v_row = dk:
// the cached latent rows of a latent attention, hundreds of channels wide, one kv head for many
// query heads). A CTA of eight warps takes AW_BM query rows, the (token, head) pairs of
// consecutive tokens of one request and up to AW_BM heads of one kv head, and walks the keys
// AW_BN at a time through two shared-memory buffers; a key tile serves as K for S = Q K^T and,
// read transposed, as V for O += P V, so each cached row is loaded once. Warp w holds rows
// 16 (w mod 4) .. +15: of S it makes the 16 keys of its half (w / 4) of the tile, the two halves
// exchange their row maxima and sums and P (bfloat16) through shared memory, and of O it keeps
// the half (w / 4) of the DV value channels in registers. Softmax state float32, as above.
#define AW_BM 64
#define AW_BN 32
#define AW_WARPS 8
#define AW_LDP (AW_BN + 8)

template <int DK, int DV>
__global__ void __launch_bounds__(AW_WARPS * 32)
attention_sink_wide_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                           long long out_stride, const bf16* __restrict__ k_cache, int page_size,
                           const int* __restrict__ block_tables, int max_blocks,
                           const int* __restrict__ positions, const int* __restrict__ seq_ids,
                           const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok, int H,
                           int Hkv, int dk, int dv, float scale_log2, int window,
                           const float* __restrict__ sinks, int n_splits, float* __restrict__ part_o,
                           float* __restrict__ part_ml, float cap_log2, float scale_over_cap) {
    constexpr int LDK = DK + AS_PAD;
    constexpr int KS = DK / 16, CHK = DK / 8, HV = DV / 2;
    constexpr int THREADS = AW_WARPS * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                // [AW_BM][LDK]
    bf16* sk = sq + AW_BM * LDK;               // [2][AW_BN][LDK]
    bf16* sp = sk + 2 * AW_BN * LDK;           // [AW_BM][AW_LDP]
    __shared__ float s_max[2][AW_BM], s_sum[2][AW_BM];
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rb = warp & 3, hf = warp >> 2;
    const int tile = gridDim.x - 1 - blockIdx.x;   // later tiles of a request read more keys
    const int G = H / Hkv;
    const int GB = G < AW_BM ? G : AW_BM;          // heads of one kv head a CTA takes
    const int hblocks = (G + GB - 1) / GB;
    const int kvh = blockIdx.y / hblocks, h0 = (blockIdx.y % hblocks) * GB;
    const int gb = G - h0 < GB ? G - h0 : GB;      // heads this CTA has
    const int tok0 = tile_tok0 ? tile_tok0[tile] : tile, ntok = tile_ntok ? tile_ntok[tile] : 1;
    const int n_rows = ntok * GB;                  // row r: token r / GB, head h0 + r % GB (if < gb)
    const int p0 = positions[tok0];
    if (p0 < 0) {                                  // a request that brings nothing: zeros out
        if (blockIdx.z == 0)
            for (int i = tid; i < n_rows * dv; i += THREADS) {
                const int r = i / dv, d = i % dv;
                if (r % GB < gb)
                    out[(size_t)(tok0 + r / GB) * out_stride + (size_t)(kvh * G + h0 + r % GB) * dv + d] =
                        __float2bfloat16_rn(0.f);
            }
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok0] * max_blocks;
    const int p_last = p0 + ntok - 1;
    const int key_lo = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int key_hi = p_last + 1;
    int t_lo = key_lo / AW_BN, t_hi = (key_hi + AW_BN - 1) / AW_BN;
    if (n_splits > 1) {
        const int per = (t_hi - t_lo + n_splits - 1) / n_splits;
        t_lo += blockIdx.z * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }
    const int chk = dk / 8;
    for (int i = tid; i < AW_BM * CHK; i += THREADS) {
        const int r = i / CHK, c = i % CHK;
        const bool ok = r < n_rows && r % GB < gb && c < chk;
        const bf16* src = ok ? q + (size_t)(tok0 + r / GB) * q_stride + (size_t)(kvh * G + h0 + r % GB) * dk + c * 8 : q;
        cp_async16(sq + r * LDK + c * 8, src, ok);
    }
    // a warp a row, the row's place in the cache worked out once for its chunks; the rows'
    // block-table reads go out together, ahead of the copies
    auto load_k = [&](int t, int buf) {
        bf16* dks = sk + buf * AW_BN * LDK;
        constexpr int RPW = AW_BN / AW_WARPS;
        size_t base[RPW];
        bool in[RPW];
#pragma unroll
        for (int x = 0; x < RPW; ++x) {
            const int j = t * AW_BN + warp + x * AW_WARPS;
            in[x] = j >= key_lo && j < key_hi;
            base[x] = 0;
            if (in[x]) {
                const int pi = j / page_size, po = j - pi * page_size;
                base[x] = (((size_t)bt[pi] * Hkv + kvh) * page_size + po) * dk;
            }
        }
#pragma unroll
        for (int x = 0; x < RPW; ++x) {
            const int r = warp + x * AW_WARPS;
#pragma unroll
            for (int c = lane; c < CHK; c += 32) {
                const bool ok = in[x] && c < chk;
                cp_async16(dks + r * LDK + c * 8, k_cache + (ok ? base[x] + c * 8 : 0), ok);
            }
        }
    };
    if (t_lo < t_hi) load_k(t_lo, 0);
    cp_async_commit();

    float o[HV / 8][4];
#pragma unroll
    for (int i = 0; i < HV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    int pos_row[2], vis_row[2], row_of[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = rb * 16 + (lane >> 2) + 8 * h;
        row_of[h] = r;
        pos_row[h] = (r < n_rows && r % GB < gb) ? p0 + r / GB : -1;   // rows beyond the tile read nothing
        vis_row[h] = (window > 0 && pos_row[h] - window + 1 > 0) ? pos_row[h] - window + 1 : 0;
    }
    const bool warp_active = rb * 16 < n_rows;

    for (int t = t_lo; t < t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_k(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kt = sk + buf * AW_BN * LDK;
        float s[2][4] = {};
        float mx[2] = {-INFINITY, -INFINITY};
        if (warp_active) {
#pragma unroll 4
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t qa[4], kb[4];
                ldmatrix_x4(qa, sq + (rb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + ks * 16 + (lane >> 4) * 8);
                ldmatrix_x4(kb, kt + (hf * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[0], qa, kb[0], kb[1]);
                mma_bf16(s[1], qa, kb[2], kb[3]);
            }
            const int kbase = t * AW_BN + hf * 16 + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = kbase + i * 8 + e;
                    const bool a = j <= pos_row[0] && j >= vis_row[0];
                    const bool c = j <= pos_row[1] && j >= vis_row[1];
                    s[i][e] = a ? as_scored(s[i][e], scale_log2, cap_log2, scale_over_cap) : -INFINITY;
                    s[i][2 + e] = c ? as_scored(s[i][2 + e], scale_log2, cap_log2, scale_over_cap) : -INFINITY;
                    mx[0] = fmaxf(mx[0], s[i][e]);
                    mx[1] = fmaxf(mx[1], s[i][2 + e]);
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                if ((lane & 3) == 0) s_max[hf][row_of[h]] = mx[h];
            }
        }
        __syncthreads();
        float corr[2] = {1.f, 1.f};
        if (warp_active) {
            float base[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mn = fmaxf(m_run[h], fmaxf(mx[h], s_max[hf ^ 1][row_of[h]]));
                base[h] = mn == -INFINITY ? 0.f : mn;      // no key seen yet: exp2(-inf - 0) = 0
                corr[h] = exp2f(m_run[h] - base[h]);
                m_run[h] = mn;
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[i][0] = exp2f(s[i][0] - base[0]);
                s[i][1] = exp2f(s[i][1] - base[0]);
                s[i][2] = exp2f(s[i][2] - base[1]);
                s[i][3] = exp2f(s[i][3] - base[1]);
                sum[0] += s[i][0] + s[i][1];
                sum[1] += s[i][2] + s[i][3];
                const int c = hf * 16 + i * 8 + (lane & 3) * 2;
                *(uint32_t*)(sp + row_of[0] * AW_LDP + c) = pack_bf16(s[i][0], s[i][1]);
                *(uint32_t*)(sp + row_of[1] * AW_LDP + c) = pack_bf16(s[i][2], s[i][3]);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
                sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
                if ((lane & 3) == 0) s_sum[hf][row_of[h]] = sum[h];
            }
        }
        __syncthreads();
        if (warp_active) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
                l_run[h] = l_run[h] * corr[h] + s_sum[0][row_of[h]] + s_sum[1][row_of[h]];
#pragma unroll
            for (int i = 0; i < HV / 8; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < AW_BN / 16; ++kk) {
                uint32_t pa[4];
                ldmatrix_x4(pa, sp + (rb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * AW_LDP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int dp = 0; dp < HV / 16; ++dp) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + hf * HV +
                                              dp * 16 + (lane >> 4) * 8);
                    mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
                    mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (!warp_active) return;
    const int col = hf * HV + (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = row_of[h];
        if (r >= n_rows || r % GB >= gb) continue;
        const int head = kvh * G + h0 + r % GB;
        float l = l_run[h];
        if (n_splits > 1) {                    // a share of the keys: the join kernel finishes
            const size_t at = ((size_t)(tok0 + r / GB) * H + head) * n_splits + blockIdx.z;
            if ((lane & 3) == 0 && hf == 0) {
                part_ml[at * 2] = m_run[h];
                part_ml[at * 2 + 1] = l;
            }
            float* po = part_o + at * dv + col;
#pragma unroll
            for (int i = 0; i < HV / 8; ++i)
                if (col + i * 8 < dv) *(float2*)(po + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
            continue;
        }
        float corr = 1.f;
        if (sinks) {                           // the sink joins the denominator last
            const float sk2 = sinks[head] * AS_LOG2E, m = m_run[h];
            const float mn = fmaxf(m, sk2);
            corr = exp2f(m - mn);
            l = l * corr + exp2f(sk2 - mn);
        }
        const float inv = l > 0.f ? corr / l : 0.f;
        bf16* dst = out + (size_t)(tok0 + r / GB) * out_stride + (size_t)head * dv + col;
#pragma unroll
        for (int i = 0; i < HV / 8; ++i)
            if (col + i * 8 < dv)
                *(uint32_t*)(dst + i * 8) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
}

// Wide rows, a step of single tokens with at most 16 query heads a kv head: the heads are the
// rows of one m16 tile that all eight warps hold. Of a 64-key tile warp w makes the scores of keys
// 8w .. 8w+7 (four accumulators that take every fourth 16-channel step, so that the chain of
// dependent products is a quarter as long), the warps exchange maxima, sums and P through
// shared memory, and of O warp w keeps DV / 8 value channels. With n_splits > 1 a CTA's share
// goes to scratch for the join kernel.
#define AWD_BN 64
#define AWD_LDP (AWD_BN + 8)

template <int DK, int DV>
__global__ void __launch_bounds__(AW_WARPS * 32)
attention_sink_wide_decode_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                                  long long out_stride, const bf16* __restrict__ k_cache, int page_size,
                                  const int* __restrict__ block_tables, int max_blocks,
                                  const int* __restrict__ positions, const int* __restrict__ seq_ids, int H,
                                  int Hkv, int dk, int dv, float scale_log2, int window,
                                  const float* __restrict__ sinks, int n_splits, float* __restrict__ part_o,
                                  float* __restrict__ part_ml, float cap_log2, float scale_over_cap) {
    constexpr int LDK = DK + AS_PAD;
    constexpr int KS = DK / 16, CHK = DK / 8, WV = DV / AW_WARPS;
    constexpr int THREADS = AW_WARPS * 32;
    static_assert(KS % 4 == 0 && WV % 16 == 0, "widths");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                // [16][LDK]
    bf16* sk = sq + 16 * LDK;                  // [2][AWD_BN][LDK]
    bf16* sp = sk + 2 * AWD_BN * LDK;          // [16][AWD_LDP]
    __shared__ float s_max[AW_WARPS][16], s_sum[AW_WARPS][16];
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tok = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = H / Hkv;
    const int p = positions[tok];
    if (p < 0) {                               // a request that brings nothing: zeros out
        if (split == 0)
            for (int i = tid; i < G * dv; i += THREADS)
                out[(size_t)tok * out_stride + (size_t)(kvh * G) * dv + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int* bt = block_tables + (size_t)seq_ids[tok] * max_blocks;
    const int key_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int key_hi = p + 1;
    int t_lo = key_lo / AWD_BN, t_hi = (key_hi + AWD_BN - 1) / AWD_BN;
    if (n_splits > 1) {
        const int per = (t_hi - t_lo + n_splits - 1) / n_splits;
        t_lo += split * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }
    const int chk = dk / 8;
    for (int i = tid; i < 16 * CHK; i += THREADS) {
        const int r = i / CHK, c = i % CHK;
        const bool ok = r < G && c < chk;
        const bf16* src = ok ? q + (size_t)tok * q_stride + (size_t)(kvh * G + r) * dk + c * 8 : q;
        cp_async16(sq + r * LDK + c * 8, src, ok);
    }
    // a warp a row, the row's place in the cache worked out once for its chunks; the rows'
    // block-table reads go out together, ahead of the copies
    auto load_k = [&](int t, int buf) {
        bf16* dks = sk + buf * AWD_BN * LDK;
        constexpr int RPW = AWD_BN / AW_WARPS;
        size_t base[RPW];
        bool in[RPW];
#pragma unroll
        for (int x = 0; x < RPW; ++x) {
            const int j = t * AWD_BN + warp + x * AW_WARPS;
            in[x] = j >= key_lo && j < key_hi;
            base[x] = 0;
            if (in[x]) {
                const int pi = j / page_size, po = j - pi * page_size;
                base[x] = (((size_t)bt[pi] * Hkv + kvh) * page_size + po) * dk;
            }
        }
#pragma unroll
        for (int x = 0; x < RPW; ++x) {
            const int r = warp + x * AW_WARPS;
#pragma unroll
            for (int c = lane; c < CHK; c += 32) {
                const bool ok = in[x] && c < chk;
                cp_async16(dks + r * LDK + c * 8, k_cache + (ok ? base[x] + c * 8 : 0), ok);
            }
        }
    };
    if (t_lo < t_hi) load_k(t_lo, 0);
    cp_async_commit();

    float o[WV / 8][4];
#pragma unroll
    for (int i = 0; i < WV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_of[2] = {lane >> 2, (lane >> 2) + 8};
    const bool row_ok[2] = {row_of[0] < G, row_of[1] < G};

    for (int t = t_lo; t < t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_k(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kt = sk + buf * AWD_BN * LDK;
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        float s2[4] = {0.f, 0.f, 0.f, 0.f}, s3[4] = {0.f, 0.f, 0.f, 0.f};
        const bf16* qrow = sq + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8;
        const bf16* krow = kt + (warp * 8 + (lane & 7)) * LDK + (lane >> 3) * 8;
#pragma unroll 3
        for (int ks = 0; ks < KS; ks += 4) {
            uint32_t qa[4][4], kb[2][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) ldmatrix_x4(qa[u], qrow + (ks + u) * 16);
            // four 8 x 8 blocks of this warp's eight keys a load: 32 channels
            ldmatrix_x4(kb[0], krow + ks * 16);
            ldmatrix_x4(kb[1], krow + (ks + 2) * 16);
            mma_bf16(s0, qa[0], kb[0][0], kb[0][1]);
            mma_bf16(s1, qa[1], kb[0][2], kb[0][3]);
            mma_bf16(s2, qa[2], kb[1][0], kb[1][1]);
            mma_bf16(s3, qa[3], kb[1][2], kb[1][3]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) { s0[e] += s2[e]; s1[e] += s3[e]; }
        float s[4], mx[2] = {-INFINITY, -INFINITY};
        const int kbase = t * AWD_BN + warp * 8 + (lane & 3) * 2;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = kbase + e;
            const bool vis = j >= key_lo && j < key_hi;
            s[e] = (vis && row_ok[0]) ? as_scored(s0[e] + s1[e], scale_log2, cap_log2, scale_over_cap) : -INFINITY;
            s[2 + e] = (vis && row_ok[1]) ? as_scored(s0[2 + e] + s1[2 + e], scale_log2, cap_log2, scale_over_cap)
                                          : -INFINITY;
            mx[0] = fmaxf(mx[0], s[e]);
            mx[1] = fmaxf(mx[1], s[2 + e]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            if ((lane & 3) == 0) s_max[warp][row_of[h]] = mx[h];
        }
        __syncthreads();
        float corr[2], sum[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mn = m_run[h];
#pragma unroll
            for (int w = 0; w < AW_WARPS; ++w) mn = fmaxf(mn, s_max[w][row_of[h]]);
            const float base = mn == -INFINITY ? 0.f : mn;      // no key seen yet: exp2(-inf - 0) = 0
            corr[h] = exp2f(m_run[h] - base);
            m_run[h] = mn;
            s[2 * h] = exp2f(s[2 * h] - base);
            s[2 * h + 1] = exp2f(s[2 * h + 1] - base);
            sum[h] = s[2 * h] + s[2 * h + 1];
            sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
            sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
            if ((lane & 3) == 0) s_sum[warp][row_of[h]] = sum[h];
            *(uint32_t*)(sp + row_of[h] * AWD_LDP + warp * 8 + (lane & 3) * 2) = pack_bf16(s[2 * h], s[2 * h + 1]);
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float l = 0.f;
#pragma unroll
            for (int w = 0; w < AW_WARPS; ++w) l += s_sum[w][row_of[h]];
            l_run[h] = l_run[h] * corr[h] + l;
        }
#pragma unroll
        for (int i = 0; i < WV / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < AWD_BN / 16; ++kk) {
            uint32_t pa[4];
            ldmatrix_x4(pa, sp + ((lane & 7) + ((lane >> 3) & 1) * 8) * AWD_LDP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int dp = 0; dp < WV / 16; ++dp) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + warp * WV +
                                          dp * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
                mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    const int col = warp * WV + (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_ok[h]) continue;
        const int head = kvh * G + row_of[h];
        float l = l_run[h];
        if (n_splits > 1) {
            const size_t at = ((size_t)tok * H + head) * n_splits + split;
            if ((lane & 3) == 0 && warp == 0) {
                part_ml[at * 2] = m_run[h];
                part_ml[at * 2 + 1] = l;
            }
            float* po = part_o + at * dv + col;
#pragma unroll
            for (int i = 0; i < WV / 8; ++i)
                if (col + i * 8 < dv) *(float2*)(po + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
            continue;
        }
        float c2 = 1.f;
        if (sinks) {
            const float sk2 = sinks[head] * AS_LOG2E, m = m_run[h];
            const float mn = fmaxf(m, sk2);
            c2 = exp2f(m - mn);
            l = l * c2 + exp2f(sk2 - mn);
        }
        const float inv = l > 0.f ? c2 / l : 0.f;
        bf16* dst = out + (size_t)tok * out_stride + (size_t)head * dv + col;
#pragma unroll
        for (int i = 0; i < WV / 8; ++i)
            if (col + i * 8 < dv)
                *(uint32_t*)(dst + i * 8) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
}

// Joins the shares of a token's keys: out = sum_s O_s 2^(m_s - m) / (sum_s l_s 2^(m_s - m) +
// 2^(sink - m)), m the largest of the maxima and the sink. A block per (token, head).
__global__ void attention_sink_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           const int* __restrict__ positions, const float* __restrict__ sinks,
                                           bf16* __restrict__ out, long long out_stride, int H, int dv,
                                           int n_splits) {
    const int tok = blockIdx.x, head = blockIdx.y;
    if (positions[tok] < 0) return;            // zeros were written by the tile kernel
    const size_t at = ((size_t)tok * H + head) * n_splits;
    const float sk2 = sinks ? sinks[head] * AS_LOG2E : -INFINITY;
    float m = sk2;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(at + s) * 2]);
    float l = sinks ? exp2f(sk2 - m) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(at + s) * 2];
        if (ms != -INFINITY) l += part_ml[(at + s) * 2 + 1] * exp2f(ms - m);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(at + s) * 2];
            if (ms != -INFINITY) a += part_o[(at + s) * dv + d] * exp2f(ms - m);
        }
        out[(size_t)tok * out_stride + (size_t)head * dv + d] = __float2bfloat16_rn(a * inv);
    }
}

TGO_API int tgo_attention_sink_supports(int H, int Hkv, int dk, int dv) {
    return (H > 0 && Hkv > 0 && H % Hkv == 0 && H / Hkv <= AS_BM && dk > 0 && dv > 0 && dk % 8 == 0 &&
            dv % 8 == 0 && dk <= 128 && dv <= 128) ? 1 : 0;
}

TGO_API int tgo_attention_sink_tile_rows() { return AS_BM; }

template <int DK, int DV>
static int launch_sink(const bf16* q, long long q_stride, bf16* out, long long out_stride,
                       const bf16* k_cache, const bf16* v_cache, int page_size, const int* block_tables,
                       int max_blocks, const int* positions, const int* seq_ids, const int* tile_tok0,
                       const int* tile_ntok, int n_tiles, int H, int Hkv, int dk, int dv, float scale,
                       int window, const float* sinks, int n_splits, float* part_o, float* part_ml,
                       float softcap, int v_row, int keep_first, const float* dist_bias, int n_dist,
                       cudaStream_t stream) {
    const float cap_log2 = softcap > 0.f ? softcap * AS_LOG2E : 0.f;
    const float scale_over_cap = softcap > 0.f ? scale / softcap : 0.f;
    const size_t smem = ((size_t)AS_BM * (DK + AS_PAD) + 2 * AS_BN * (DK + AS_PAD) + 2 * AS_BN * (DV + AS_PAD)) *
                        sizeof(bf16);
    int rc;
    if (!tile_tok0 && H / Hkv <= 16) {
        // single tokens, few heads a kv head: the form whose four warps share each key tile
        // (its shared memory also holds the warps' O, [4][16][DV] floats, at the join)
        size_t dsm = ((size_t)16 * (DK + AS_PAD) + 2 * AS_BN * (DK + AS_PAD) + 2 * AS_BN * (DV + AS_PAD)) * sizeof(bf16);
        const size_t need = (size_t)16 * (DK + AS_PAD) * sizeof(bf16) + (size_t)4 * 16 * DV * sizeof(float);
        if (dsm < need) dsm = need;
        auto dec = attention_sink_decode_kernel<DK, DV>;
        if (dsm > 48 * 1024) cudaFuncSetAttribute(dec, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm);
        rc = tgo_launch_pdl(dec, dim3(n_tiles, Hkv, n_splits), dim3(128), dsm, stream, q, q_stride, out,
                            out_stride, k_cache, v_cache, page_size, block_tables, max_blocks, positions, seq_ids,
                            H, Hkv, dk, dv, scale * AS_LOG2E, window, sinks, n_splits, part_o, part_ml,
                            cap_log2, scale_over_cap, v_row, keep_first, dist_bias, n_dist);
    } else {
        auto kernel = attention_sink_kernel<DK, DV>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<dim3(n_tiles, Hkv, n_splits), AS_WARPS * 32, smem, stream>>>(
            q, q_stride, out, out_stride, k_cache, v_cache, page_size, block_tables, max_blocks, positions,
            seq_ids, tile_tok0, tile_ntok, H, Hkv, dk, dv, scale * AS_LOG2E, window, sinks, n_splits, part_o,
            part_ml, cap_log2, scale_over_cap, v_row, keep_first, dist_bias, n_dist);
        rc = launch_status();
    }
    if (rc || n_splits <= 1) return rc;
    attention_sink_join_kernel<<<dim3(n_tiles, H), 64, 0, stream>>>(part_o, part_ml, positions, sinks, out,
                                                                   out_stride, H, dv, n_splits);
    return launch_status();
}

// q [T, >= H dk] and out [T, >= H dv] bfloat16 views with unit column stride, 16-byte aligned
// rows; tile lists int32 [n_tiles] (at most tgo_attention_sink_tile_rows() / (H / Hkv) tokens
// of one request each) or null with n_tiles = T; then n_splits > 1 cuts every token's keys
// over as many CTAs, with scratch part_o float32 [T, H, n_splits, dv] and part_ml float32
// [T, H, n_splits, 2].
TGO_API int tgo_attention_sink(const void* q, long long q_stride, void* out, long long out_stride,
                               const void* k_cache, const void* v_cache, int page_size,
                               const int* block_tables, int max_blocks, const int* positions,
                               const int* seq_ids, const int* tile_tok0, const int* tile_ntok,
                               int n_tiles, int H, int Hkv, int dk, int dv, float scale, int window,
                               const float* sinks, int n_splits, float* part_o, float* part_ml,
                               float softcap, int v_row, int keep_first, const float* dist_bias,
                               int n_dist, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (v_row <= 0) v_row = dv;
    if (v_row < dv || (v_row % 8) || !(softcap >= 0.f) || keep_first < 0 || (dist_bias && n_dist <= 0))
        return TGO_E_BAD_ARG;
    if (window == 0) keep_first = 0;
    if (!tgo_attention_sink_supports(H, Hkv, dk, dv) || page_size <= 0 || max_blocks <= 0 || window < 0 ||
        Hkv > 65535 || (q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)out % 4) ||
        ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16) || (!tile_tok0) != (!tile_ntok) ||
        n_splits < 1 || n_splits > 65535 ||
        (n_splits > 1 && (tile_tok0 || !part_o || !part_ml || ((uintptr_t)part_o % 8))))
        return TGO_E_BAD_ARG;
#define AS_GO(DK, DV) launch_sink<DK, DV>((const bf16*)q, q_stride, (bf16*)out, out_stride,              \
                                          (const bf16*)k_cache, (const bf16*)v_cache, page_size,          \
                                          block_tables, max_blocks, positions, seq_ids, tile_tok0,        \
                                          tile_ntok, n_tiles, H, Hkv, dk, dv, scale, window, sinks,   \
                                          n_splits, part_o, part_ml, softcap, v_row, keep_first, dist_bias, \
                                          n_dist, stream)
    if (dk <= 64) return dv <= 64 ? AS_GO(64, 64) : AS_GO(64, 128);
    return dv <= 64 ? AS_GO(128, 64) : AS_GO(128, 128);
#undef AS_GO
}

// ---- wide rows, values inside the key rows
TGO_API int tgo_attention_sink_wide_supports(int H, int Hkv, int dk, int dv) {
    return (H > 0 && Hkv > 0 && H % Hkv == 0 && dk > 0 && dv > 0 && dv <= dk && dk % 8 == 0 && dv % 8 == 0 &&
            dk <= 576 && dv <= 512) ? 1 : 0;
}

// Tokens of one request a tile holds at most, for `group` query heads a kv head.
TGO_API int tgo_attention_sink_wide_tile_tokens(int group) {
    return group >= AW_BM ? 1 : AW_BM / group;
}

template <int DK, int DV>
static int launch_sink_wide(const bf16* q, long long q_stride, bf16* out, long long out_stride,
                            const bf16* k_cache, int page_size, const int* block_tables, int max_blocks,
                            const int* positions, const int* seq_ids, const int* tile_tok0,
                            const int* tile_ntok, int n_tiles, int H, int Hkv, int dk, int dv, float scale,
                            int window, const float* sinks, int n_splits, float* part_o, float* part_ml,
                            float softcap, cudaStream_t stream) {
    const float cap_log2 = softcap > 0.f ? softcap * AS_LOG2E : 0.f;
    const float scale_over_cap = softcap > 0.f ? scale / softcap : 0.f;
    const size_t smem = ((size_t)(AW_BM + 2 * AW_BN) * (DK + AS_PAD) + (size_t)AW_BM * AW_LDP) * sizeof(bf16);
    const int G = H / Hkv, GB = G < AW_BM ? G : AW_BM;
    int rc;
    if (!tile_tok0 && G <= 16) {               // single tokens, few heads a kv head: all warps on one m16 tile
        const size_t dsm = ((size_t)(16 + 2 * AWD_BN) * (DK + AS_PAD) + (size_t)16 * AWD_LDP) * sizeof(bf16);
        auto dec = attention_sink_wide_decode_kernel<DK, DV>;
        if (dsm > 48 * 1024) cudaFuncSetAttribute(dec, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm);
        rc = tgo_launch_pdl(dec, dim3(n_tiles, Hkv, n_splits), dim3(AW_WARPS * 32), dsm, stream, q, q_stride, out,
                            out_stride, k_cache, page_size, block_tables, max_blocks, positions, seq_ids, H, Hkv,
                            dk, dv, scale * AS_LOG2E, window, sinks, n_splits, part_o, part_ml, cap_log2,
                            scale_over_cap);
        if (rc || n_splits <= 1) return rc;
        attention_sink_join_kernel<<<dim3(n_tiles, H), 128, 0, stream>>>(part_o, part_ml, positions, sinks, out,
                                                                        out_stride, H, dv, n_splits);
        return launch_status();
    }
    auto kernel = attention_sink_wide_kernel<DK, DV>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rc = tgo_launch_pdl(kernel, dim3(n_tiles, Hkv * ((G + GB - 1) / GB), n_splits), dim3(AW_WARPS * 32), smem,
                            stream, q, q_stride, out, out_stride, k_cache, page_size, block_tables, max_blocks,
                            positions, seq_ids, tile_tok0, tile_ntok, H, Hkv, dk, dv, scale * AS_LOG2E, window,
                            sinks, n_splits, part_o, part_ml, cap_log2, scale_over_cap);
    if (rc || n_splits <= 1) return rc;
    attention_sink_join_kernel<<<dim3(n_tiles, H), 128, 0, stream>>>(part_o, part_ml, positions, sinks, out,
                                                                    out_stride, H, dv, n_splits);
    return launch_status();
}

// As tgo_attention_sink for key rows up to 576 wide whose first dv (up to 512) channels are the
// values: one cache plane [page, kv head, offset, dk]. Tile lists hold at most
// tgo_attention_sink_wide_tile_tokens(H / Hkv) tokens of one request each.
TGO_API int tgo_attention_sink_wide(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* k_cache, int page_size, const int* block_tables,
                                    int max_blocks, const int* positions, const int* seq_ids,
                                    const int* tile_tok0, const int* tile_ntok, int n_tiles, int H, int Hkv,
                                    int dk, int dv, float scale, int window, const float* sinks,
                                    int n_splits, float* part_o, float* part_ml, float softcap,
                                    cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (!tgo_attention_sink_wide_supports(H, Hkv, dk, dv) || !(softcap >= 0.f) || page_size <= 0 ||
        max_blocks <= 0 || window < 0 || (q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) ||
        ((uintptr_t)out % 4) || ((uintptr_t)k_cache % 16) || (!tile_tok0) != (!tile_ntok) || n_splits < 1 ||
        n_splits > 65535 || (n_splits > 1 && (tile_tok0 || !part_o || !part_ml || ((uintptr_t)part_o % 8))))
        return TGO_E_BAD_ARG;
#define AW_GO(DK, DV) launch_sink_wide<DK, DV>((const bf16*)q, q_stride, (bf16*)out, out_stride,             \
                                               (const bf16*)k_cache, page_size, block_tables, max_blocks,   \
                                               positions, seq_ids, tile_tok0, tile_ntok, n_tiles, H, Hkv,   \
                                               dk, dv, scale, window, sinks, n_splits, part_o, part_ml,     \
                                               softcap, stream)
    if (dk <= 192 && dv <= 128) return AW_GO(192, 128);
    if (dk <= 320 && dv <= 256) return AW_GO(320, 256);
    return AW_GO(576, 512);
#undef AW_GO
}
