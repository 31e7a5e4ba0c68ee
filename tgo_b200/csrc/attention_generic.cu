// Paged causal attention, one warp per (token, head), any head size up to 256 (rows whose
// values lie inside the keys: up to 1152) and any
// storage type. It is the float32 path's attention and the fallback of the bfloat16
// path for head sizes that the tensor-core kernels do not take.
//
// The query at position p of request b reads keys lo..p, lo = max(0, p - window + 1)
// (window 0: lo = 0), through the request's block table. Keys are taken 32 at a time
// starting at lo, so the order of every sum depends on (p, window) alone: the result
// for a position is bit-identical however the tokens were cut into steps or batched.
//
// Keys are dh wide and values dv wide (two cache planes with rows of their own when they
// differ). With `sinks` (float32, one number per query head) the softmax's denominator also
// holds exp(sink_h): a key that is always seen, is not scaled and has no value.
// `softcap` > 0 bounds every score: s <- softcap * tanh(s / softcap), after the scale.
// A value row starts `v_row` elements after the one before it: dv for a plane of values; the
// key rows' width when a value is the first dv channels of its key row (one cache plane that
// serves as both, v_cache = k_cache).
// `keep_first` > 0 (with a window): the first keep_first keys of the request stay visible to
// every later query, at their true positions, beside the window. The keys are then walked as
// one list (the kept ones that lie before the window, then the window), 32 at a time, so the
// order of the sums still depends on (p, window, keep_first) alone.
// `dist_bias` (float32 [n_dist][H]): dist_bias[min(p - j, n_dist - 1)][h] is added to the
// scaled score of key j, unscaled (a learned bias by distance).
#include "common.cuh"

#define AG_MAX_DH 256            // rows up to this wide take the instance with 8 sums a lane
#define AG_MAX_WIDE 640          // wider ones, up to this, the instance with 20
#define AG_MAX_WIDEST 1152       // and up to this (a latent of 1024 with its rotated part), 36
#define AG_WARPS 4

template <typename T, int NACC>
__global__ void attention_generic_kernel(
    const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
    int H, int Hkv, int dh, int dv, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    int page_size, const int* __restrict__ block_tables, int max_blocks,
    const int* __restrict__ seq_ids, const int* __restrict__ positions, float scale, int window,
    const float* __restrict__ sinks, float softcap, int v_row, int keep_first,
    const float* __restrict__ dist_bias, int n_dist) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * AG_WARPS + warp;
    if (h >= H) return;
    float* qs = smem + warp * dh;
    const int p = positions[t];
    const int b = p >= 0 ? seq_ids[t] : 0;
    const int kvh = h / (H / Hkv);
    const int* bt = block_tables + (size_t)b * max_blocks;
    const T* qv = q + (size_t)t * q_stride + (size_t)h * dh;
    for (int i = lane; i < dh; i += 32) qs[i] = to_f32(qv[i]);
    __syncwarp();

    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

    const int nkept = keep_first < lo ? keep_first : lo;       // kept keys that lie before the window
    const int nkeys = p >= 0 ? nkept + (p - lo + 1) : 0;
    for (int vbase = 0; vbase < nkeys; vbase += 32) {
        const int vj = vbase + lane;
        const int j = vj < nkept ? vj : lo + (vj - nkept);
        const int nvalid = (nkeys - vbase) < 32 ? (nkeys - vbase) : 32;
        float s = -INFINITY;
        if (vj < nkeys) {
            const int page = bt[j / page_size];
            const T* kr = k_cache + (((size_t)page * Hkv + kvh) * page_size + (j % page_size)) * dh;
            float a = 0.f;
            for (int d = 0; d < dh; ++d) a += qs[d] * to_f32(kr[d]);
            s = a * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
            if (dist_bias) s += dist_bias[(size_t)((p - j) < n_dist ? (p - j) : n_dist - 1) * H + h];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);          // m = -inf the first time: corr = 0
        const float w = vj < nkeys ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(w);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        for (int jj = 0; jj < nvalid; ++jj) {
            const float wj = __shfl_sync(0xffffffffu, w, jj);
            const int kj = (vbase + jj) < nkept ? vbase + jj : lo + (vbase + jj - nkept);
            const int page = bt[kj / page_size];
            const T* vr = v_cache + (((size_t)page * Hkv + kvh) * page_size + (kj % page_size)) * v_row;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] += wj * to_f32(vr[d]);
            }
        }
        m = m_new;
    }
    if (sinks && p >= 0) {                         // the sink joins the denominator last
        const float sk = sinks[h];
        const float m_new = fmaxf(m, sk);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    }
    T* o = out + (size_t)t * out_stride + (size_t)h * dv;
    const float inv = l > 0.f ? 1.f / l : 0.f;     // position < 0: no keys, zeros out
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) o[d] = from_f32<T>(acc[i] * inv);
    }
}

TGO_API int tgo_attention_generic(const void* q, long long q_stride, void* out,
                                  long long out_stride, int dtype, int T, int H, int Hkv, int dh, int dv,
                                  const void* k_cache, const void* v_cache, int page_size,
                                  const int* block_tables, int max_blocks, const int* seq_ids,
                                  const int* positions, float scale, int window,
                                  const float* sinks, float softcap, int v_row, int keep_first,
                                  const float* dist_bias, int n_dist, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (v_row <= 0) v_row = dv;
    if (dh <= 0 || dh > AG_MAX_WIDEST || dv <= 0 || dv > AG_MAX_WIDEST || H <= 0 || Hkv <= 0 || H % Hkv ||
        page_size <= 0 || max_blocks <= 0 || window < 0 || v_row < dv || !(softcap >= 0.f) || keep_first < 0 ||
        (dist_bias && n_dist <= 0))
        return TGO_E_BAD_ARG;
    const bool wide = dv > AG_MAX_DH, widest = dv > AG_MAX_WIDE;
    const dim3 grid(T, (H + AG_WARPS - 1) / AG_WARPS);
    const size_t smem = (size_t)AG_WARPS * dh * sizeof(float);
#define AG_GO(TT, NACC)                                                                            \
    attention_generic_kernel<TT, NACC><<<grid, AG_WARPS * 32, smem, stream>>>(                         \
        (const TT*)q, q_stride, (TT*)out, out_stride, H, Hkv, dh, dv, (const TT*)k_cache,              \
        (const TT*)v_cache, page_size, block_tables, max_blocks, seq_ids, positions, scale, window,   \
        sinks, softcap, v_row, keep_first, dist_bias, n_dist)
    if (dtype == TGO_BF16) {
        if (widest) AG_GO(bf16, AG_MAX_WIDEST / 32); else if (wide) AG_GO(bf16, AG_MAX_WIDE / 32); else AG_GO(bf16, AG_MAX_DH / 32);
    } else if (dtype == TGO_F32) {
        if (widest) AG_GO(float, AG_MAX_WIDEST / 32); else if (wide) AG_GO(float, AG_MAX_WIDE / 32); else AG_GO(float, AG_MAX_DH / 32);
    } else
        return TGO_E_BAD_ARG;
#undef AG_GO
    return launch_status();
}
