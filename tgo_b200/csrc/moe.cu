// A routed feed-forward (mixture of experts): every token goes to the `top` experts with the
// largest router logits, weighted by the softmax over those logits alone.
//
//   route      logits = Wr x + br in float32 (Wr, br float32; x in the storage type), the top
//              experts (ties: the lower index), their weights, and a count per expert
//   plan       expert e's (token, choice) pairs get places offsets[e] .. offsets[e+1]-1; the
//              places are cut into row tiles of one expert each
//   scatter    pair -> place (within an expert the order is whatever the atomics give; a
//              pair's result does not depend on its place)
//   up         hidden[place] = act(x Wg_e^T) * (x Wu_e^T) for the token of the pair at `place`
//   down       y[pair] = hidden[place] Wd_e^T, float32
//   combine    out[t] = sum_j weight[t][j] y[t top + j] (+ extra[t]), j in order, all float32
//
// The products are tiled: float32 storage takes plain-FMA tiles with float32 sums over k in
// order; bfloat16 storage takes mma.sync m16n8k16 tiles (float32 accumulators) fed by cp.async
// through two shared-memory buffers, when the widths are multiples of 8 (16-byte chunks), and
// the plain tiles otherwise. Either way a row's result does not depend on which tile or batch
// it falls in.
//
// Variants, each a parameter: `score_mode` 1 takes the softmax over ALL router logits; the choice
// is by that score plus a per-expert `correction`, the weights are the chosen experts' scores
// (without the correction) divided by their sum (+ 1e-20). The last router outputs past the
// `E_real` experts that have matrices are identity experts: their output is the token's input
// row itself; they get no place and no tile, the combine adds weight * x for them. One more
// router row after all experts (`gate_out`) gives a logistic gate per token that multiplies
// `extra` in the combine. Experts without a gate matrix (wg null) are W_down act(W_up x);
// activation 3 is the square of relu.
#include "mma_sync.cuh"

#define MOE_TM 64
#define MOE_TN 64
#define MOE_TK 16

// ------------------------------------------------------------------------------- route
// A block of four warps per MOE_RT tokens: warp w takes experts w, w + 4, ... and makes their
// logits for all the block's tokens at once (a row of Wr is read once per block), lanes over
// the width; then warp t picks token t's experts.
#define MOE_RT 4
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ wr,
                 const float* __restrict__ br, int Tn, int d, int E, int top, int* __restrict__ ids,
                 float* __restrict__ wts, int* __restrict__ counts, int score_mode,
                 const float* __restrict__ correction, int E_real, float* __restrict__ gate_out) {
    extern __shared__ float smem[];                      // [MOE_RT][E + 1] logits, [MOE_RT][E] scores
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * MOE_RT;
    const int nt = Tn - t0 < MOE_RT ? Tn - t0 : MOE_RT;
    const int rows = E + (gate_out ? 1 : 0), ld = E + 1;
    for (int e = warp; e < rows; e += 4) {
        const float* w = wr + (size_t)e * d;
        float a[MOE_RT];
#pragma unroll
        for (int j = 0; j < MOE_RT; ++j) a[j] = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float wv = w[i];
#pragma unroll
            for (int j = 0; j < MOE_RT; ++j)
                if (j < nt) a[j] = fmaf(wv, to_f32(x[(size_t)(t0 + j) * x_stride + i]), a[j]);
        }
#pragma unroll
        for (int j = 0; j < MOE_RT; ++j) {
            const float v = warp_sum(a[j]);
            if (lane == 0) smem[j * ld + e] = v + ((br && e < E) ? br[e] : 0.f);
        }
    }
    __syncthreads();
    if (warp >= nt) return;
    const int t = t0 + warp;
    float* lg = smem + (size_t)warp * ld;
    if (gate_out && lane == 0) gate_out[t] = 1.f / (1.f + expf(-lg[E]));
    float first = 0.f, sum = 0.f, mine = 0.f;
    int mine_e = 0;
    if (score_mode == 1) {
        // scores: the softmax over every logit; the choice adds the correction
        float* sc = smem + (size_t)MOE_RT * ld + (size_t)warp * E;
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
        mx = warp_max(mx);
        float den = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float w = expf(lg[e] - mx);
            sc[e] = w;
            den += w;
        }
        den = warp_sum(den);
        for (int e = lane; e < E; e += 32) {
            const float sv = sc[e] / den;
            sc[e] = sv;
            lg[e] = sv + (correction ? correction[e] : 0.f);
        }
        __syncwarp();
        for (int j = 0; j < top; ++j) {
            float best = -INFINITY;
            int be = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = lg[e];
                if (v > best || (v == best && e < be)) { best = v; be = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
            }
            const float w = sc[be];
            sum += w;
            if (lane == j) { mine = w; mine_e = be; }
            if (lane == 0) lg[be] = -INFINITY;
            __syncwarp();
        }
        if (lane < top) {
            ids[(size_t)t * top + lane] = mine_e;
            wts[(size_t)t * top + lane] = mine / (sum + 1e-20f);
            if (mine_e < E_real) atomicAdd(&counts[mine_e], 1);
        }
        return;
    }
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = lg[e];
            if (v > best || (v == best && e < be)) { best = v; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
        }
        if (j == 0) first = best;
        const float w = expf(best - first);
        sum += w;
        if (lane == j) { mine = w; mine_e = be; }
        if (lane == 0) lg[be] = -INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        ids[(size_t)t * top + lane] = mine_e;
        wts[(size_t)t * top + lane] = mine / sum;
        if (mine_e < E_real) atomicAdd(&counts[mine_e], 1);
    }
}

// -------------------------------------------------------------------------------- plan
// One thread: offsets [E + 1], tiles (expert, first place, rows) and their count in
// tile_info[0]; the fill counters go back to zero.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                int* __restrict__ fill, int* __restrict__ tile_info,
                                int* __restrict__ tiles, int max_tiles) {
    pdl_wait();
    if (threadIdx.x || blockIdx.x) return;
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
        offsets[e] = at;
        fill[e] = 0;
        const int c = counts[e];
        for (int r = 0; r < c && nt < max_tiles; r += MOE_TM) {
            tiles[3 * nt] = e;
            tiles[3 * nt + 1] = at + r;
            tiles[3 * nt + 2] = c - r < MOE_TM ? c - r : MOE_TM;
            ++nt;
        }
        at += c;
    }
    offsets[E] = at;
    tile_info[0] = nt;
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, int pairs,
                                   const int* __restrict__ offsets, int* __restrict__ fill,
                                   int* __restrict__ perm, int* __restrict__ place, int E_real) {
    pdl_wait();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pairs) return;
    const int e = ids[p];
    if (e >= E_real) { place[p] = -1; return; }          // an identity expert: no matrices, no place
    const int at = offsets[e] + atomicAdd(&fill[e], 1);
    perm[at] = p;
    place[p] = at;
}

// ----------------------------------------------------------------------------- products
__device__ __forceinline__ float moe_act(float z, int act) {
    if (act == 1) return z > 0.f ? z : 0.f;
    if (act == 3) return z > 0.f ? z * z : 0.f;
    if (act == 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.f + expf(-z));
}

// hidden[place][f] = act(x_tok . Wg[e][f]) * (x_tok . Wu[e][f]); Wg, Wu [E, ff, d]. Without a
// gate matrix (wg null): act(x_tok . Wu[e][f]).
template <typename T>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ wg,
              const T* __restrict__ wu, T* __restrict__ hidden, int d, int ff, int top, int act,
              const int* __restrict__ perm, const int* __restrict__ tile_info,
              const int* __restrict__ tiles) {
    __shared__ float xs[MOE_TK][MOE_TM + 4];
    __shared__ float gs[MOE_TK][MOE_TN + 4];
    __shared__ float us[MOE_TK][MOE_TN + 4];
    __shared__ int toks[MOE_TM];
    pdl_wait();
    if ((int)blockIdx.y >= tile_info[0]) return;
    const int e = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * MOE_TN;
    if (threadIdx.x < MOE_TM) toks[threadIdx.x] = threadIdx.x < rows ? perm[r0 + threadIdx.x] / top : -1;
    __syncthreads();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* wge = wg + (size_t)e * ff * d;
    const T* wue = wu + (size_t)e * ff * d;
    float ag[4][4], au[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) ag[i][j] = au[i][j] = 0.f;
    for (int k0 = 0; k0 < d; k0 += MOE_TK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int row = idx / MOE_TK, kk = idx % MOE_TK;
            const int gk = k0 + kk, gn = n0 + row;
            const int tok = toks[row];
            xs[kk][row] = (tok >= 0 && gk < d) ? to_f32(x[(size_t)tok * x_stride + gk]) : 0.f;
            const bool in = gn < ff && gk < d;
            gs[kk][row] = (in && wg) ? to_f32(wge[(size_t)gn * d + gk]) : 0.f;
            us[kk][row] = in ? to_f32(wue[(size_t)gn * d + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float a[4], g[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { g[j] = gs[kk][tx * 4 + j]; u[j] = us[kk][tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ag[i][j] = fmaf(a[i], g[j], ag[i][j]);
                    au[i][j] = fmaf(a[i], u[j], au[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = ty * 4 + i;
        if (row >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < ff)
                hidden[(size_t)(r0 + row) * ff + gn] =
                    from_f32<T>(wg ? moe_act(ag[i][j], act) * au[i][j] : moe_act(au[i][j], act));
        }
    }
}

// y[pair][n] = hidden[place] . Wd[e][n]; Wd [E, d, ff]; y float32 [pairs, d].
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ hidden, const T* __restrict__ wd, float* __restrict__ y, int d,
                int ff, const int* __restrict__ perm, const int* __restrict__ tile_info,
                const int* __restrict__ tiles) {
    __shared__ float hs[MOE_TK][MOE_TM + 4];
    __shared__ float ws[MOE_TK][MOE_TN + 4];
    pdl_wait();
    if ((int)blockIdx.y >= tile_info[0]) return;
    const int e = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * MOE_TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* wde = wd + (size_t)e * d * ff;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < ff; k0 += MOE_TK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int row = idx / MOE_TK, kk = idx % MOE_TK;
            const int gk = k0 + kk, gn = n0 + row;
            hs[kk][row] = (row < rows && gk < ff) ? to_f32(hidden[(size_t)(r0 + row) * ff + gk]) : 0.f;
            ws[kk][row] = (gn < d && gk < ff) ? to_f32(wde[(size_t)gn * ff + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = hs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = ty * 4 + i;
        if (row >= rows) continue;
        const int pair = perm[r0 + row];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < d) y[(size_t)pair * d + gn] = acc[i][j];
        }
    }
}

// ------------------------------------------------------------- products on the tensor cores
// A tile of up to 64 rows of one expert by 64 columns; four warps, warp w owns rows 16w..16w+15
// and all 64 columns. UP: A rows are x rows gathered by token, B is Wg[e] and Wu[e] ([N, K]
// each), the result act(gate) * up goes to hidden[place] in bfloat16. MODE 1 is that; MODE 2
// is the form without a gate, B is Wu[e] alone and the result act(up). MODE 0: A rows are
// hidden[place], B is Wd[e], the result goes to y[pair] in float32.
#define MT_BK 64
#define MT_LD (MT_BK + 8)
#define MT_STAGES 3

template <int MODE>
__global__ void __launch_bounds__(128)
moe_tc_kernel(const bf16* __restrict__ a, long long a_stride, const bf16* __restrict__ w0,
              const bf16* __restrict__ w1, bf16* __restrict__ hidden, float* __restrict__ y, int N,
              int K, int top, int act, const int* __restrict__ perm,
              const int* __restrict__ tile_info, const int* __restrict__ tiles) {
    extern __shared__ __align__(16) unsigned char moe_smem[];
    typedef bf16 (*Tile)[MOE_TM][MT_LD];
    Tile As = (Tile)moe_smem;                                        // [MT_STAGES][64][MT_LD]
    Tile B0 = (Tile)(moe_smem + sizeof(bf16) * MT_STAGES * MOE_TM * MT_LD);
    Tile B1 = (Tile)(moe_smem + sizeof(bf16) * 2 * MT_STAGES * MOE_TM * MT_LD);   // UP only
    __shared__ int src_row[MOE_TM];
    constexpr bool UP = MODE != 0, GATED = MODE == 1;
    pdl_wait();
    if ((int)blockIdx.y >= tile_info[0]) return;
    const int e = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * MOE_TN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MOE_TM) src_row[tid] = tid < rows ? (UP ? perm[r0 + tid] / top : r0 + tid) : -1;
    __syncthreads();
    const bf16* w0e = w0 + (size_t)e * N * K;
    const bf16* w1e = GATED ? w1 + (size_t)e * N * K : nullptr;
    auto load = [&](int k0, int buf) {
        // 64 rows x 8 chunks of 8 per operand
        for (int i = tid; i < MOE_TM * (MT_BK / 8); i += 128) {
            const int r = i >> 3, c = i & 7;
            const int k = k0 + c * 8;
            const int sr = src_row[r];
            const bool oka = sr >= 0 && k < K;
            cp_async16(&As[buf][r][c * 8], oka ? a + (size_t)sr * a_stride + k : a, oka);
            const bool okb = n0 + r < N && k < K;
            cp_async16(&B0[buf][r][c * 8], okb ? w0e + (size_t)(n0 + r) * K + k : w0, okb);
            if (GATED) cp_async16(&B1[buf][r][c * 8], okb ? w1e + (size_t)(n0 + r) * K + k : w0, okb);
        }
    };
    float c0[MOE_TN / 8][4], c1[GATED ? MOE_TN / 8 : 1][4];
#pragma unroll
    for (int i = 0; i < MOE_TN / 8; ++i) c0[i][0] = c0[i][1] = c0[i][2] = c0[i][3] = 0.f;
#pragma unroll
    for (int i = 0; i < (GATED ? MOE_TN / 8 : 1); ++i) c1[i][0] = c1[i][1] = c1[i][2] = c1[i][3] = 0.f;
    const int steps = (K + MT_BK - 1) / MT_BK;
#pragma unroll
    for (int p = 0; p < MT_STAGES - 1; ++p) {
        if (p < steps) load(p * MT_BK, p);
        cp_async_commit();
    }
    const bool warp_active = warp * 16 < rows;
    for (int st = 0; st < steps; ++st) {
        const int buf = st % MT_STAGES;
        cp_async_wait<MT_STAGES - 2>();                   // this step's tiles have landed
        __syncthreads();                                  // and the buffer of step st - 1 is free
        if (st + MT_STAGES - 1 < steps) load((st + MT_STAGES - 1) * MT_BK, (st + MT_STAGES - 1) % MT_STAGES);
        cp_async_commit();
        if (warp_active) {
#pragma unroll
            for (int ks = 0; ks < MT_BK / 16; ++ks) {
                uint32_t fa[4];
                ldmatrix_x4(fa, &As[buf][warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
                for (int np = 0; np < MOE_TN / 16; ++np) {
                    uint32_t fb[4];
                    ldmatrix_x4(fb, &B0[buf][np * 16 + (lane & 7) + (lane >> 4) * 8][ks * 16 + ((lane >> 3) & 1) * 8]);
                    mma_bf16(c0[2 * np], fa, fb[0], fb[1]);
                    mma_bf16(c0[2 * np + 1], fa, fb[2], fb[3]);
                    if (GATED) {
                        ldmatrix_x4(fb, &B1[buf][np * 16 + (lane & 7) + (lane >> 4) * 8][ks * 16 + ((lane >> 3) & 1) * 8]);
                        mma_bf16(c1[2 * np], fa, fb[0], fb[1]);
                        mma_bf16(c1[2 * np + 1], fa, fb[2], fb[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    if (!warp_active) return;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + (lane >> 2) + 8 * h;
        if (row >= rows) continue;
        const int pair = UP ? 0 : perm[r0 + row];
#pragma unroll
        for (int i = 0; i < MOE_TN / 8; ++i) {
            const int col = n0 + i * 8 + (lane & 3) * 2;
            if (col >= N) continue;                       // N is even: col + 1 < N too
            if (UP) {
                const float v0 = moe_act(c0[i][2 * h], act) * (GATED ? c1[GATED ? i : 0][2 * h] : 1.f);
                const float v1 = moe_act(c0[i][2 * h + 1], act) * (GATED ? c1[GATED ? i : 0][2 * h + 1] : 1.f);
                *(uint32_t*)(hidden + (size_t)(r0 + row) * N + col) = pack_bf16(v0, v1);
            } else {
                *(float2*)(y + (size_t)pair * N + col) = make_float2(c0[i][2 * h], c0[i][2 * h + 1]);
            }
        }
    }
}

// out[t][c] = sum_j wts[t][j] y[t top + j][c] + extra_gate[t] * extra[t][c]; a pair whose
// expert is an identity expert (ids >= E_real; `ids` null: there are none) contributes
// wts * x[t][c] instead.
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts,
                                   const float* __restrict__ extra, float* __restrict__ out, int d,
                                   int top, const int* __restrict__ ids, int E_real,
                                   const T* __restrict__ x, long long x_stride,
                                   const float* __restrict__ extra_gate) {
    pdl_wait();
    const int t = blockIdx.x;
    const float eg = extra_gate ? extra_gate[t] : 1.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float a = 0.f;
        for (int j = 0; j < top; ++j) {
            const size_t pair = (size_t)t * top + j;
            const float v = (ids && ids[pair] >= E_real) ? to_f32(x[(size_t)t * x_stride + c]) : y[pair * d + c];
            a = fmaf(wts[pair], v, a);
        }
        if (extra) a = fmaf(eg, extra[(size_t)t * d + c], a);
        out[(size_t)t * d + c] = a;
    }
}

TGO_API int tgo_moe_tile_rows() { return MOE_TM; }

// ids, place int32 [T top]; wts float32 [T top]; counts, fill int32 [E]; offsets int32 [E + 1];
// perm int32 [T top]; tile_info int32 [1]; tiles int32 [3 max_tiles].
TGO_API int tgo_moe_route(const void* x, long long x_stride, int dtype, const float* wr,
                          const float* br, int T, int d, int E, int top, int* ids, float* wts,
                          int* counts, int* fill, int* offsets, int* perm, int* place,
                          int* tile_info, int* tiles, int max_tiles, int score_mode,
                          const float* correction, int E_real, float* gate_out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || E <= 0 || E > 2048 || top <= 0 || top > 32 || top > E || max_tiles <= 0 ||
        E_real < 0 || E_real > E || score_mode < 0 || score_mode > 1)
        return TGO_E_BAD_ARG;
    int rc = E_real ? (int)cudaMemsetAsync(counts, 0, sizeof(int) * E_real, stream) : 0;
    if (rc) return rc;
    const size_t smem = (size_t)MOE_RT * (2 * E + 1) * sizeof(float);
    if (smem > 48 * 1024) {                              // more than about 1500 router outputs
        cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (dtype == TGO_BF16)
        moe_route_kernel<bf16><<<(T + MOE_RT - 1) / MOE_RT, 128, smem, stream>>>((const bf16*)x, x_stride, wr, br, T, d, E,
                                                                  top, ids, wts, counts, score_mode, correction, E_real, gate_out);
    else if (dtype == TGO_F32)
        moe_route_kernel<float><<<(T + MOE_RT - 1) / MOE_RT, 128, smem, stream>>>((const float*)x, x_stride, wr, br, T, d,
                                                                   E, top, ids, wts, counts, score_mode, correction, E_real, gate_out);
    else
        return TGO_E_BAD_ARG;
    if ((rc = launch_status())) return rc;
    rc = tgo_launch_pdl(moe_plan_kernel, dim3(1), dim3(32), 0, stream, (const int*)counts, E_real, offsets, fill,
                        tile_info, tiles, max_tiles);
    if (rc) return rc;
    const int pairs = T * top;
    return tgo_launch_pdl(moe_scatter_kernel, dim3((pairs + 255) / 256), dim3(256), 0, stream,
                          (const int*)ids, pairs, (const int*)offsets, fill, perm, place, E_real);
}

// x [T, d] rows (stride x_stride); wg, wu [E, ff, d]; wd [E, d, ff]; hidden [T top, ff] in the
// storage type; y float32 [T top, d]; extra float32 [T, d] or null; out float32 [T, d].
TGO_API int tgo_moe_experts(const void* x, long long x_stride, int dtype, const void* wg,
                            const void* wu, const void* wd, void* hidden, float* y,
                            const float* wts, const float* extra, float* out, int T, int d, int ff,
                            int top, int act, const int* perm, const int* tile_info,
                            const int* tiles, int max_tiles, const int* ids, int E_real,
                            const float* extra_gate, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || ff <= 0 || top <= 0 || max_tiles <= 0 || max_tiles > 65535 || act < 0 || act > 3)
        return TGO_E_BAD_ARG;
#define MOE_COMBINE(TT)                                                                            \
    tgo_launch_pdl(moe_combine_kernel<TT>, dim3(T), dim3(256), 0, stream, (const float*)y, wts, extra, out, \
                   d, top, ids, E_real, (const TT*)x, x_stride, extra_gate)
    const dim3 g1((ff + MOE_TN - 1) / MOE_TN, max_tiles), g2((d + MOE_TN - 1) / MOE_TN, max_tiles);
    int rc;
    const bool chunks = d % 8 == 0 && ff % 8 == 0 && x_stride % 8 == 0 && (uintptr_t)x % 16 == 0 &&
                        (uintptr_t)wg % 16 == 0 && (uintptr_t)wu % 16 == 0 && (uintptr_t)wd % 16 == 0 &&
                        (uintptr_t)hidden % 16 == 0 && (uintptr_t)y % 8 == 0;
    if (dtype == TGO_BF16 && chunks) {
        const size_t tile = sizeof(bf16) * MT_STAGES * MOE_TM * MT_LD;
        static bool asked = false;
        if (!asked) {
            cudaFuncSetAttribute(moe_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(3 * tile));
            cudaFuncSetAttribute(moe_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * tile));
            cudaFuncSetAttribute(moe_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * tile));
            asked = true;
        }
        if (wg)
            rc = tgo_launch_pdl(moe_tc_kernel<1>, g1, dim3(128), 3 * tile, stream, (const bf16*)x, x_stride,
                                (const bf16*)wg, (const bf16*)wu, (bf16*)hidden, (float*)nullptr, ff, d, top, act,
                                perm, tile_info, tiles);
        else
            rc = tgo_launch_pdl(moe_tc_kernel<2>, g1, dim3(128), 2 * tile, stream, (const bf16*)x, x_stride,
                                (const bf16*)wu, (const bf16*)nullptr, (bf16*)hidden, (float*)nullptr, ff, d, top,
                                act, perm, tile_info, tiles);
        if (rc) return rc;
        rc = tgo_launch_pdl(moe_tc_kernel<0>, g2, dim3(128), 2 * tile, stream, (const bf16*)hidden, (long long)ff,
                            (const bf16*)wd, (const bf16*)nullptr, (bf16*)nullptr, y, d, ff, top, act, perm,
                            tile_info, tiles);
        if (rc) return rc;
        return MOE_COMBINE(bf16);
    }
    if (dtype == TGO_BF16) {
        rc = tgo_launch_pdl(moe_up_kernel<bf16>, g1, dim3(256), 0, stream, (const bf16*)x, x_stride,
                            (const bf16*)wg, (const bf16*)wu, (bf16*)hidden, d, ff, top, act, perm, tile_info,
                            tiles);
        if (rc) return rc;
        rc = tgo_launch_pdl(moe_down_kernel<bf16>, g2, dim3(256), 0, stream, (const bf16*)hidden,
                            (const bf16*)wd, y, d, ff, perm, tile_info, tiles);
        if (rc) return rc;
        return MOE_COMBINE(bf16);
    }
    if (dtype != TGO_F32) return TGO_E_BAD_ARG;
    rc = tgo_launch_pdl(moe_up_kernel<float>, g1, dim3(256), 0, stream, (const float*)x, x_stride,
                        (const float*)wg, (const float*)wu, (float*)hidden, d, ff, top, act, perm, tile_info,
                        tiles);
    if (rc) return rc;
    rc = tgo_launch_pdl(moe_down_kernel<float>, g2, dim3(256), 0, stream, (const float*)hidden,
                        (const float*)wd, y, d, ff, perm, tile_info, tiles);
    if (rc) return rc;
    return MOE_COMBINE(float);
#undef MOE_COMBINE
}
