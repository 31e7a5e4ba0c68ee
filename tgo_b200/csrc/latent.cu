// Pieces of attention over a compressed (latent) cache: every token keeps one row
// [c (rank), r (rope width)] in a single cache plane, c the normed latent that keys and values
// are expanded from and r a rotated key part shared by all heads. With the expansion matrices
// folded into the query and the output ("absorbed"), attention over that plane is attention
// with ONE key/value head whose key is the whole row and whose value is its first `rank`
// channels:
//
//   score_h(i, j) = ((W_uk_h^T q_h,nope(i)) . c(j) + q_h,rope(i) . r(j)) * scale
//   out_h(i)      = W_uv_h (sum_j w_h(i, j) c(j))
//
// Here: the row's making (norm of c, rotation of r, cache write), the per-head products that
// fold W_uk into the query and W_uv into the output, and the rotation of a slice of every
// head into another tensor. Norm, rotation and every sum are float32.
#include "common.cuh"

// ---------------------------------------------------------- latent row -> cache plane
// A block a token. kv [T, >= rank + width] (strided): the first `rank` channels are divided
// by their root mean square and multiplied by gain; of the last `width` the first `rot` are
// rotated (pairs i, i + rot/2, or 2i, 2i + 1 if `interleaved`) by the token's row of `rope`
// (cos then sin, [T, rot]). The row goes to cache[page][offset][rank + width] at `slots[t]`.
template <typename T>
__global__ void __launch_bounds__(128)
latent_row_cache_kernel(const T* __restrict__ kv, long long kv_stride, int rank, int width,
                        const float* __restrict__ gain, float eps, const float* __restrict__ rope,
                        int rot, int interleaved, const int* __restrict__ slots, T* __restrict__ cache,
                        int page_size) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.x;
    const int slot = slots[t];
    const T* src = kv + (size_t)t * kv_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float x = to_f32(src[i]);
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    if (slot < 0) return;
    const float r = rsqrtf(ss / (float)rank + eps);
    T* dst = cache + (size_t)slot * (rank + width);       // pages are contiguous: slot = page * page_size + offset
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        dst[i] = from_f32<T>((to_f32(src[i]) * r) * gain[i]);
    const int half = rot / 2;
    const float* cs = rope ? rope + (size_t)t * rot : nullptr;
    for (int i = threadIdx.x; i < width - half; i += blockDim.x) {
        if (i < half) {
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float xa = to_f32(src[rank + a]), xb = to_f32(src[rank + b]);
            const float c = cs ? cs[i] : 1.f, sn = cs ? cs[half + i] : 0.f;
            dst[rank + a] = from_f32<T>(xa * c - xb * sn);
            dst[rank + b] = from_f32<T>(xb * c + xa * sn);
        } else {
            dst[rank + i + half] = src[rank + i + half];
        }
    }
}

TGO_API int tgo_latent_row_cache(const void* kv, long long kv_stride, int dtype, int T, int rank,
                                 int width, const float* gain, float eps, const float* rope, int rot,
                                 int interleaved, const int* slots, void* cache, int page_size,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rank <= 0 || width < 0 || rot < 0 || rot > width || (rot & 1) || !gain || !slots || !cache ||
        page_size <= 0)
        return TGO_E_BAD_ARG;
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(latent_row_cache_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)kv,
                              kv_stride, rank, width, gain, eps, rope, rot, interleaved, slots, (bf16*)cache,
                              page_size);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(latent_row_cache_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)kv,
                              kv_stride, rank, width, gain, eps, rope, rot, interleaved, slots, (float*)cache,
                              page_size);
    return TGO_E_BAD_ARG;
}

// ------------------------------------------- a slice of every head, rotated, into another tensor
// dst[t, h * dst_head + dst_off + i] = rotated src[t, h * src_head + src_off + i], i < width:
// the first `rot` channels of the slice are rotated, the rest copied. One warp a (token, head).
template <typename T>
__global__ void rope_slice_kernel(const T* __restrict__ src, long long src_stride, int src_head, int src_off,
                                  T* __restrict__ dst, long long dst_stride, int dst_head, int dst_off, int H,
                                  int width, const float* __restrict__ rope, int rot, int interleaved) {
    pdl_wait();
    const int t = blockIdx.x;
    const int h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= H) return;
    const T* s = src + (size_t)t * src_stride + (size_t)h * src_head + src_off;
    T* d = dst + (size_t)t * dst_stride + (size_t)h * dst_head + dst_off;
    const int half = rot / 2;
    const float* cs = rope ? rope + (size_t)t * rot : nullptr;
    for (int i = lane; i < width - half; i += 32) {
        if (i < half) {
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float xa = to_f32(s[a]), xb = to_f32(s[b]);
            const float c = cs ? cs[i] : 1.f, sn = cs ? cs[half + i] : 0.f;
            d[a] = from_f32<T>(xa * c - xb * sn);
            d[b] = from_f32<T>(xb * c + xa * sn);
        } else {
            d[i + half] = s[i + half];
        }
    }
}

TGO_API int tgo_rope_slice(const void* src, long long src_stride, int src_head, int src_off, void* dst,
                           long long dst_stride, int dst_head, int dst_off, int dtype, int T, int H,
                           int width, const float* rope, int rot, int interleaved, cudaStream_t stream) {
    if (T <= 0 || width <= 0) return 0;
    if (H <= 0 || rot < 0 || rot > width || (rot & 1) || H > 4 * 65535) return TGO_E_BAD_ARG;
    const dim3 grid(T, (H + 3) / 4), block(128);
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(rope_slice_kernel<bf16>, grid, block, 0, stream, (const bf16*)src, src_stride,
                              src_head, src_off, (bf16*)dst, dst_stride, dst_head, dst_off, H, width, rope, rot,
                              interleaved);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(rope_slice_kernel<float>, grid, block, 0, stream, (const float*)src, src_stride,
                              src_head, src_off, (float*)dst, dst_stride, dst_head, dst_off, H, width, rope,
                              rot, interleaved);
    return TGO_E_BAD_ARG;
}

// --------------------------------------------------------------- a product per head
// y[t, h * y_head + n] = sum_k x[t, h * x_head + k] * w[h][n][k],  n < N, k < K: every head has
// a matrix of its own, w [H][N][K] contiguous. A block makes HL_TOK tokens by HL_N outputs of
// one head; a thread sums one output's k in ascending order for one or several tokens, so an
// output's bits do not depend on what else is in the step. HL_N is 64, or 16 when that gives
// too few blocks to fill the device (few tokens, few outputs a head). x, y: rows with unit
// column stride.
#define HL_TOK 16
#define HL_K 32

template <typename T, int HL_N>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, long long x_stride, int x_head, const T* __restrict__ w,
                   T* __restrict__ y, long long y_stride, int y_head, int Tn, int N, int K) {
    __shared__ float xs[HL_TOK][HL_K + 1];
    __shared__ float ws[HL_N][HL_K + 1];
    pdl_wait();
    const int t0 = blockIdx.x * HL_TOK, h = blockIdx.y, n0 = blockIdx.z * HL_N;
    constexpr int TG = 256 / HL_N, PER = HL_TOK / TG;              // tokens tg, tg + TG, ...
    const int nl = threadIdx.x % HL_N, tg = threadIdx.x / HL_N;
    const T* wh = w + (size_t)h * N * K;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HL_K) {
        __syncthreads();
        for (int i = threadIdx.x; i < HL_TOK * HL_K; i += 256) {
            const int r = i / HL_K, c = i % HL_K;
            const bool ok = t0 + r < Tn && k0 + c < K;
            xs[r][c] = ok ? to_f32(x[(size_t)(t0 + r) * x_stride + (size_t)h * x_head + k0 + c]) : 0.f;
        }
        for (int i = threadIdx.x; i < HL_N * HL_K; i += 256) {
            const int r = i / HL_K, c = i % HL_K;
            const bool ok = n0 + r < N && k0 + c < K;
            ws[r][c] = ok ? to_f32(wh[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < HL_K; ++c) {
            const float wv = ws[nl][c];
#pragma unroll
            for (int i = 0; i < PER; ++i) acc[i] += xs[tg + TG * i][c] * wv;
        }
    }
    if (n0 + nl >= N) return;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int t = t0 + tg + TG * i;
        if (t < Tn) y[(size_t)t * y_stride + (size_t)h * y_head + n0 + nl] = from_f32<T>(acc[i]);
    }
}

// Up to 16 rows (a step of a few single tokens; with more, walking the rows costs more than the
// tiles below) and K up to 512: a warp an output of one head. A lane holds
// the weights k = lane, lane + 32, ... of its output in registers and walks the tokens, four at
// a time; the lanes' partial sums are joined by shuffles in a fixed order, so an output's bits
// depend on nothing but its own row. The weights are read once, 64 bytes a warp and load.
#define HLF_PER 16
template <typename T>
__global__ void __launch_bounds__(256)
head_linear_few_kernel(const T* __restrict__ x, long long x_stride, int x_head, const T* __restrict__ w,
                       T* __restrict__ y, long long y_stride, int y_head, int Tn, int N, int K) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), h = blockIdx.y;
    if (n >= N) return;
    const T* wr = w + ((size_t)h * N + n) * K;
    float wv[HLF_PER];
#pragma unroll
    for (int i = 0; i < HLF_PER; ++i) wv[i] = lane + 32 * i < K ? to_f32(wr[lane + 32 * i]) : 0.f;
    for (int t0 = 0; t0 < Tn; t0 += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u < Tn) {
                const T* xr = x + (size_t)(t0 + u) * x_stride + (size_t)h * x_head;
#pragma unroll
                for (int i = 0; i < HLF_PER; ++i)
                    if (lane + 32 * i < K) acc[u] += wv[i] * to_f32(xr[lane + 32 * i]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float a = warp_sum(acc[u]);
            if (lane == 0 && t0 + u < Tn) y[(size_t)(t0 + u) * y_stride + (size_t)h * y_head + n] = from_f32<T>(a);
        }
    }
}

TGO_API int tgo_head_linear(const void* x, long long x_stride, int x_head, const void* w, void* y,
                            long long y_stride, int y_head, int dtype, int T, int H, int N, int K,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || N <= 0 || K <= 0 || H > 65535) return TGO_E_BAD_ARG;
    if (T <= 16 && K <= 32 * HLF_PER && (N + 7) / 8 <= 0x7fffffff) {
        const dim3 fgrid((N + 7) / 8, H), fblock(256);
        if (dtype == TGO_BF16)
            return tgo_launch_pdl(head_linear_few_kernel<bf16>, fgrid, fblock, 0, stream, (const bf16*)x, x_stride,
                                  x_head, (const bf16*)w, (bf16*)y, y_stride, y_head, T, N, K);
        if (dtype == TGO_F32)
            return tgo_launch_pdl(head_linear_few_kernel<float>, fgrid, fblock, 0, stream, (const float*)x,
                                  x_stride, x_head, (const float*)w, (float*)y, y_stride, y_head, T, N, K);
        return TGO_E_BAD_ARG;
    }
    const long long blocks64 = (long long)((T + HL_TOK - 1) / HL_TOK) * H * ((N + 63) / 64);
    const int hn = blocks64 < 600 ? 16 : 64;
    const dim3 grid((T + HL_TOK - 1) / HL_TOK, H, (N + hn - 1) / hn), block(256);
    if (grid.z > 65535) return TGO_E_BAD_ARG;
#define HL_GO(TT, NN)                                                                                       \
    return tgo_launch_pdl(head_linear_kernel<TT, NN>, grid, block, 0, stream, (const TT*)x, x_stride, x_head, \
                          (const TT*)w, (TT*)y, y_stride, y_head, T, N, K)
    if (dtype == TGO_BF16) {
        if (hn == 16) HL_GO(bf16, 16);
        HL_GO(bf16, 64);
    }
    if (dtype == TGO_F32) {
        if (hn == 16) HL_GO(float, 16);
        HL_GO(float, 64);
    }
#undef HL_GO
    return TGO_E_BAD_ARG;
}
