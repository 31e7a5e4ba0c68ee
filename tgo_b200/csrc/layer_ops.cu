// Small per-row kernels of layers that norm a sublayer's OUTPUT and scale it per channel
// before the residual add, of feed-forwards with another gate than SiLU, of mixers that
// norm, blend and store values, of gated per-head output norms, and the soft cap on logits.
// All sums, norms and the residual stream are float32; T is the storage type of activations.
#include "common.cuh"

// ------------------------------------------------------------ float32 stream -> activations
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ h, T* __restrict__ out, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(h[i]);
}

TGO_API int tgo_cast_rows(const float* h, void* out, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype != TGO_BF16) return TGO_E_BAD_ARG;
    return tgo_launch_pdl(cast_rows_kernel<bf16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                          stream, h, (bf16*)out, (size_t)n);
}

// ------------------------------------------- h += scale * gain * group_rmsnorm(y)  (+ copy)
// grid (rows, groups): a block norms one group of one row: the d / groups channels of the
// group are divided by sqrt(mean of their squares + eps), multiplied by gain and by the
// per-channel scale (if given), and added to the stream. If `act` is given the new stream
// values are also written there in the activation type: the next sublayer's input.
template <typename TY, typename TA>
__global__ void group_norm_scale_add_kernel(float* __restrict__ h, const TY* __restrict__ y,
                                            const float* __restrict__ gain,
                                            const float* __restrict__ scale, float eps, int d,
                                            int groups, TA* __restrict__ act, int keep) {
    extern __shared__ float ykeep[];          // the group's y, if `keep`: read from memory once
    __shared__ float scratch[33];
    pdl_wait();
    const int width = d / groups;
    const size_t base = (size_t)blockIdx.x * d + (size_t)blockIdx.y * width;
    const int c0 = blockIdx.y * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32(y[base + i]);
        if (keep) ykeep[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = ((keep ? ykeep[i] : to_f32(y[base + i])) * r) * gain[c0 + i];
        if (scale) v *= scale[c0 + i];
        const float s = h[base + i] + v;
        h[base + i] = s;
        if (act) act[base + i] = from_f32<TA>(s);
    }
}

// The same with 16-byte accesses: float32 y, four channels a thread and step; needs
// width % 4 == 0 and 16-byte aligned rows. y stays in shared memory between the two passes.
__global__ void group_norm_scale_add_vec_kernel(float* __restrict__ h, const float* __restrict__ y,
                                                const float* __restrict__ gain,
                                                const float* __restrict__ scale, float eps, int d,
                                                int groups, bf16* __restrict__ act) {
    extern __shared__ float4 ykeep4[];
    __shared__ float scratch[33];
    pdl_wait();
    const int width = d / groups, w4 = width / 4;
    const size_t base = (size_t)blockIdx.x * d + (size_t)blockIdx.y * width;
    const int c0 = blockIdx.y * width;
    const float4* y4 = (const float4*)(y + base);
    float ss = 0.f;
    for (int i = threadIdx.x; i < w4; i += blockDim.x) {
        const float4 v = y4[i];
        ykeep4[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)width + eps);
    float4* h4 = (float4*)(h + base);
    const float4* g4 = (const float4*)(gain + c0);
    const float4* s4 = scale ? (const float4*)(scale + c0) : nullptr;
    for (int i = threadIdx.x; i < w4; i += blockDim.x) {
        const float4 v = ykeep4[i], g = g4[i];
        float4 o = make_float4((v.x * r) * g.x, (v.y * r) * g.y, (v.z * r) * g.z, (v.w * r) * g.w);
        if (s4) {
            const float4 sc = s4[i];
            o.x *= sc.x; o.y *= sc.y; o.z *= sc.z; o.w *= sc.w;
        }
        float4 s = h4[i];
        s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
        h4[i] = s;
        if (act) {
            uint2 p;
            __nv_bfloat162 lo = __floats2bfloat162_rn(s.x, s.y), hi = __floats2bfloat162_rn(s.z, s.w);
            p.x = *(uint32_t*)&lo;
            p.y = *(uint32_t*)&hi;
            *(uint2*)(act + base + 4 * i) = p;
        }
    }
}

TGO_API int tgo_group_norm_scale_add(float* h, const void* y, int y_dtype, const float* gain,
                                     const float* scale, float eps, int groups, void* act,
                                     int act_dtype, int T, int d, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || groups <= 0 || d % groups) return TGO_E_BAD_ARG;
    if (act && act_dtype != TGO_BF16) return TGO_E_BAD_ARG;
    const int width = d / groups;
    const dim3 grid(T, groups), block(width >= 1024 ? 256 : width >= 256 ? 128 : 64);
    const int keep = (size_t)width * 4 <= 40 * 1024 ? 1 : 0;
    const size_t smem = keep ? (size_t)width * 4 : 0;
    const bool aligned = width % 4 == 0 && !((uintptr_t)h & 15) && !((uintptr_t)y & 15) &&
                         !((uintptr_t)gain & 15) && !((uintptr_t)scale & 15) && !((uintptr_t)act & 7);
    if (y_dtype == TGO_F32 && keep && aligned)
        return tgo_launch_pdl(group_norm_scale_add_vec_kernel, grid, block, smem, stream, h,
                              (const float*)y, gain, scale, eps, d, groups, (bf16*)act);
    if (y_dtype == TGO_BF16)
        return tgo_launch_pdl(group_norm_scale_add_kernel<bf16, bf16>, grid, block, smem, stream, h,
                              (const bf16*)y, gain, scale, eps, d, groups, (bf16*)act, keep);
    if (y_dtype == TGO_F32)
        return tgo_launch_pdl(group_norm_scale_add_kernel<float, bf16>, grid, block, smem, stream, h,
                              (const float*)y, gain, scale, eps, d, groups, (bf16*)act, keep);
    return TGO_E_BAD_ARG;
}

// --------------------------------------------- out = gain * group_rmsnorm(h[rows]) (no add)
template <typename TO>
__global__ void group_norm_rows_kernel(const float* __restrict__ h, const int* __restrict__ rows,
                                       const float* __restrict__ gain, float eps, int d,
                                       int groups, TO* __restrict__ out) {
    __shared__ float scratch[33];
    pdl_wait();
    const int width = d / groups;
    const size_t row = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    const float* x = h + row * d + (size_t)blockIdx.y * width;
    TO* o = out + (size_t)blockIdx.x * d + (size_t)blockIdx.y * width;
    const int c0 = blockIdx.y * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss += x[i] * x[i];
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        o[i] = from_f32<TO>((x[i] * r) * gain[c0 + i]);
}

TGO_API int tgo_group_norm_rows(const float* h, const int* rows, const float* gain, float eps,
                                int groups, void* out, int out_dtype, int n, int d,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || groups <= 0 || d % groups) return TGO_E_BAD_ARG;
    const int width = d / groups;
    const dim3 grid(n, groups), block(width >= 1024 ? 256 : width >= 256 ? 128 : 64);
    if (out_dtype == TGO_BF16)
        return tgo_launch_pdl(group_norm_rows_kernel<bf16>, grid, block, 0, stream, h, rows, gain,
                              eps, d, groups, (bf16*)out);
    if (out_dtype == TGO_F32)
        return tgo_launch_pdl(group_norm_rows_kernel<float>, grid, block, 0, stream, h, rows, gain,
                              eps, d, groups, (float*)out);
    return TGO_E_BAD_ARG;
}

// --------------------------------------------------------------- soft cap: x <- c tanh(x / c)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

TGO_API int tgo_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return TGO_E_BAD_ARG;
    return tgo_launch_pdl(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                          x, (size_t)n, cap);
}

// ------------------------------------------------------- out = act(gate) * up, act by code
#define TGO_ACT_SILU 0
#define TGO_ACT_RELU 1
#define TGO_ACT_GELU_TANH 2
__device__ __forceinline__ float gate_act(float g, int act) {
    if (act == TGO_ACT_RELU) return fmaxf(g, 0.f);
    if (act == TGO_ACT_GELU_TANH)
        return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.f + expf(-g));
}

// `bias` (float32 [2f], laid out like a row of gu, or null) is added to the gate and up
// columns in float32 before the activation.
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int f,
                                 int interleaved, int act, const float* __restrict__ bias) {
    pdl_wait();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= f) return;
    const T* row = gu + (size_t)blockIdx.y * 2 * f;
    const int gi = interleaved ? (j / 8) * 16 + (j % 8) : j;
    const int ui = interleaved ? gi + 8 : f + j;
    const float g = to_f32(row[gi]) + (bias ? bias[gi] : 0.f);
    const float u = to_f32(row[ui]) + (bias ? bias[ui] : 0.f);
    out[(size_t)blockIdx.y * f + j] = from_f32<T>(gate_act(g, act) * u);
}

// bfloat16, eight columns a thread (16-byte accesses): needs f % 8 == 0. The results are rounded
// to bfloat16, so SiLU takes the hardware's exponential and division.
template <int ACT, bool BIAS>
__global__ void gated_act_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int f,
                                        int interleaved, const float* __restrict__ bias) {
    pdl_wait();
    const int j8 = blockIdx.x * blockDim.x + threadIdx.x;       // which group of eight columns
    if (j8 * 8 >= f) return;
    const bf16* row = gu + (size_t)blockIdx.y * 2 * f;
    const int gi = interleaved ? j8 * 16 : j8 * 8, ui = interleaved ? j8 * 16 + 8 : f + j8 * 8;
    const uint4 g4 = *(const uint4*)(row + gi);
    const uint4 u4 = *(const uint4*)(row + ui);
    float bg[8] = {}, bu[8] = {};
    if (BIAS) {                                                  // gi, ui are multiples of 8: 32-byte aligned
        *(float4*)bg = *(const float4*)(bias + gi);
        *(float4*)(bg + 4) = *(const float4*)(bias + gi + 4);
        *(float4*)bu = *(const float4*)(bias + ui);
        *(float4*)(bu + 4) = *(const float4*)(bias + ui + 4);
    }
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&g4;
    const __nv_bfloat162* u2 = (const __nv_bfloat162*)&u4;
    uint4 o4;
    __nv_bfloat162* o2 = (__nv_bfloat162*)&o4;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        float2 g = __bfloat1622float2(g2[x]), u = __bfloat1622float2(u2[x]);
        g.x += bg[2 * x]; g.y += bg[2 * x + 1];
        u.x += bu[2 * x]; u.y += bu[2 * x + 1];
        float ax, ay;
        if (ACT == 0) {
            ax = __fdividef(g.x, 1.f + __expf(-g.x));
            ay = __fdividef(g.y, 1.f + __expf(-g.y));
        } else {
            ax = gate_act(g.x, ACT);
            ay = gate_act(g.y, ACT);
        }
        o2[x] = __floats2bfloat162_rn(ax * u.x, ay * u.y);
    }
    *(uint4*)(out + (size_t)blockIdx.y * f + j8 * 8) = o4;
}

template <int ACT>
static int gated_act_x8(const bf16* gu, bf16* out, int T, int f, int interleaved, const float* bias,
                        cudaStream_t stream) {
    const dim3 grid((f / 8 + 255) / 256, T), block(256);
    if (bias)
        return tgo_launch_pdl(gated_act_bf16x8_kernel<ACT, true>, grid, block, 0, stream, gu, out, f, interleaved,
                              bias);
    return tgo_launch_pdl(gated_act_bf16x8_kernel<ACT, false>, grid, block, 0, stream, gu, out, f, interleaved,
                          bias);
}

TGO_API int tgo_gated_act(const void* gate_up, void* out, int dtype, int T, int f,
                          int interleaved, int act, const float* bias, cudaStream_t stream) {
    if (T <= 0 || f <= 0) return 0;
    if (act < 0 || act > 2 || (interleaved && f % 8)) return TGO_E_BAD_ARG;
    const dim3 grid((f + 255) / 256, T), block(256);
    if (dtype == TGO_BF16 && f % 8 == 0 && !((uintptr_t)gate_up & 15) && !((uintptr_t)out & 15) &&
        !((uintptr_t)bias & 15)) {
        if (act == 0) return gated_act_x8<0>((const bf16*)gate_up, (bf16*)out, T, f, interleaved, bias, stream);
        if (act == 1) return gated_act_x8<1>((const bf16*)gate_up, (bf16*)out, T, f, interleaved, bias, stream);
        return gated_act_x8<2>((const bf16*)gate_up, (bf16*)out, T, f, interleaved, bias, stream);
    }
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(gated_act_kernel<bf16>, grid, block, 0, stream, (const bf16*)gate_up,
                              (bf16*)out, f, interleaved, act, bias);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(gated_act_kernel<float>, grid, block, 0, stream,
                              (const float*)gate_up, (float*)out, f, interleaved, act, bias);
    return TGO_E_BAD_ARG;
}

// ------------------------------------------ values: per-head norm, blend, store in the cache
// One warp per (token, kv head). v is divided by its root mean square over vdim (if `norm`);
// mode 1 also writes the result (float32) to `shared` [T, Hkv * vdim] for later layers;
// mode 2 reads that row and blends: v <- (1 - lambda) v + lambda shared. What comes out is
// stored at the token's slot of the cache plane [page][kv head][offset][vdim]; slot < 0
// stores nothing.
#define VN_WARPS 4
template <typename T>
__global__ void value_norm_share_cache_kernel(const T* __restrict__ v, long long v_stride, int Hkv,
                                              int vdim, int norm, float eps,
                                              const float* __restrict__ lambda,
                                              float* __restrict__ shared, int mode,
                                              const int* __restrict__ slots,
                                              T* __restrict__ v_cache, int page_size) {
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * VN_WARPS + warp;
    if (head >= Hkv) return;
    const T* src = v + (size_t)t * v_stride + (size_t)head * vdim;
    float r = 1.f;
    if (norm) {
        float ss = 0.f;
        for (int i = lane; i < vdim; i += 32) {
            const float x = to_f32(src[i]);
            ss += x * x;
        }
        ss = warp_sum(ss);
        r = rsqrtf(ss / (float)vdim + eps);
    }
    const int slot = slots[t];
    T* dst = slot >= 0 ? v_cache + (((size_t)(slot / page_size) * Hkv + head) * page_size +
                                    (slot % page_size)) * vdim
                       : nullptr;
    float* sh = shared ? shared + ((size_t)t * Hkv + head) * vdim : nullptr;
    const float lam = mode == 2 ? lambda[0] : 0.f;
    for (int i = lane; i < vdim; i += 32) {
        float x = to_f32(src[i]) * r;
        if (mode == 1) sh[i] = x;
        if (mode == 2) x = (1.f - lam) * x + lam * sh[i];
        if (dst) dst[i] = from_f32<T>(x);
    }
}

TGO_API int tgo_value_norm_share_cache(const void* v, long long v_stride, int dtype, int T, int Hkv,
                                       int vdim, int norm, float eps, const float* lambda,
                                       float* shared, int mode, const int* slots, void* v_cache,
                                       int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (Hkv <= 0 || vdim <= 0 || page_size <= 0 || mode < 0 || mode > 2 ||
        (mode != 0 && !shared) || (mode == 2 && !lambda) || !slots || !v_cache)
        return TGO_E_BAD_ARG;
    const dim3 grid(T, (Hkv + VN_WARPS - 1) / VN_WARPS), block(VN_WARPS * 32);
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(value_norm_share_cache_kernel<bf16>, grid, block, 0, stream,
                              (const bf16*)v, v_stride, Hkv, vdim, norm, eps, lambda, shared, mode,
                              slots, (bf16*)v_cache, page_size);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(value_norm_share_cache_kernel<float>, grid, block, 0, stream,
                              (const float*)v, v_stride, Hkv, vdim, norm, eps, lambda, shared,
                              mode, slots, (float*)v_cache, page_size);
    return TGO_E_BAD_ARG;
}

// ---------------------------- out = o / rms(o over each head) * silu(gate), per (token, head)
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate,
                                      long long gate_stride, T* __restrict__ out, int heads,
                                      int vdim, float eps) {
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * VN_WARPS + warp;
    if (head >= heads) return;
    const float* x = o + ((size_t)t * heads + head) * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)vdim + eps);
    const T* g = gate ? gate + (size_t)t * gate_stride + (size_t)head * vdim : nullptr;
    T* y = out + ((size_t)t * heads + head) * vdim;
    for (int i = lane; i < vdim; i += 32) {
        float v = x[i] * r;
        if (g) {
            const float z = to_f32(g[i]);
            v *= z / (1.f + expf(-z));
        }
        y[i] = from_f32<T>(v);
    }
}

TGO_API int tgo_head_norm_gate(const float* o, const void* gate, long long gate_stride, void* out,
                               int dtype, int T, int heads, int vdim, float eps,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || vdim <= 0) return TGO_E_BAD_ARG;
    const dim3 grid(T, (heads + VN_WARPS - 1) / VN_WARPS), block(VN_WARPS * 32);
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(head_norm_gate_kernel<bf16>, grid, block, 0, stream, o,
                              (const bf16*)gate, gate_stride, (bf16*)out, heads, vdim, eps);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(head_norm_gate_kernel<float>, grid, block, 0, stream, o,
                              (const float*)gate, gate_stride, (float*)out, heads, vdim, eps);
    return TGO_E_BAD_ARG;
}

// ---------------------------------------------------------------------------------------
// Gated group norm of a recurrent mixer's float32 output: the row is cut into `groups` equal
// consecutive parts, each divided by sqrt(mean of its squares + eps), times the gain (null:
// none). The gate g (a column view in the activation type; null: none) goes through
// `gate_act` (1 SiLU, 2 logistic) and multiplies either the input of the norm
// (`gate_first`) or its result. A block per (token, group).
__device__ __forceinline__ float gate_value(float z, int act) {
    const float s = 1.f / (1.f + expf(-z));
    return act == 1 ? z * s : act == 2 ? s : z;
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                        const float* __restrict__ gain, T* __restrict__ out, int width, int groups,
                        float eps, int gate_act, int gate_first) {
    __shared__ float scratch[33];
    pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y;
    const int n = width / groups;
    const float* x = o + (size_t)t * width + (size_t)g * n;
    const T* gz = gate ? gate + (size_t)t * gate_stride + (size_t)g * n : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i];
        if (gz && gate_first) v *= gate_value(to_f32(gz[i]), gate_act);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)n + eps);
    T* y = out + (size_t)t * width + (size_t)g * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[i];
        if (gz && gate_first) v *= gate_value(to_f32(gz[i]), gate_act);
        v *= r;
        if (gain) v *= gain[g * n + i];
        if (gz && !gate_first) v *= gate_value(to_f32(gz[i]), gate_act);
        y[i] = from_f32<T>(v);
    }
}

// Groups of up to 512 channels: a warp a (token, group), the group's values in registers between
// the sum of squares and the scaling, no block-wide sum. Four warps a block.
#define GGN_PER 16
template <typename T>
__global__ void __launch_bounds__(128)
gated_group_norm_warp_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                             const float* __restrict__ gain, T* __restrict__ out, int width, int groups,
                             float eps, int gate_act, int gate_first, long long pairs) {
    pdl_wait();
    const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= pairs) return;
    const int lane = threadIdx.x & 31;
    const long long t = w / groups;
    const int g = (int)(w % groups);
    const int n = width / groups;
    const float* x = o + (size_t)t * width + (size_t)g * n;
    const T* gz = gate ? gate + (size_t)t * gate_stride + (size_t)g * n : nullptr;
    float v[GGN_PER], z[GGN_PER];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < GGN_PER; ++u) {
        const int i = lane + 32 * u;
        v[u] = i < n ? x[i] : 0.f;
        z[u] = (gz && i < n) ? gate_value(to_f32(gz[i]), gate_act) : 1.f;
        if (gate_first) v[u] *= z[u];
        ss += v[u] * v[u];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)n + eps);
    T* y = out + (size_t)t * width + (size_t)g * n;
#pragma unroll
    for (int u = 0; u < GGN_PER; ++u) {
        const int i = lane + 32 * u;
        if (i < n) {
            float a = v[u] * r;
            if (gain) a *= gain[g * n + i];
            if (!gate_first) a *= z[u];
            y[i] = from_f32<T>(a);
        }
    }
}

TGO_API int tgo_gated_group_norm(const float* o, const void* gate, long long gate_stride,
                                 const float* gain, void* out, int dtype, int T, int width,
                                 int groups, float eps, int gate_act, int gate_first,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (width <= 0 || groups <= 0 || width % groups || groups > 65535 || gate_act < 0 || gate_act > 2)
        return TGO_E_BAD_ARG;
    const int n = width / groups;
    const long long pairs = (long long)T * groups;
    if (n <= 32 * GGN_PER && (pairs + 3) / 4 <= 0x7fffffffLL) {
        const dim3 wgrid((unsigned)((pairs + 3) / 4)), wblock(128);
        if (dtype == TGO_BF16)
            return tgo_launch_pdl(gated_group_norm_warp_kernel<bf16>, wgrid, wblock, 0, stream, o,
                                  (const bf16*)gate, gate_stride, gain, (bf16*)out, width, groups, eps, gate_act,
                                  gate_first, pairs);
        if (dtype == TGO_F32)
            return tgo_launch_pdl(gated_group_norm_warp_kernel<float>, wgrid, wblock, 0, stream, o,
                                  (const float*)gate, gate_stride, gain, (float*)out, width, groups, eps,
                                  gate_act, gate_first, pairs);
        return TGO_E_BAD_ARG;
    }
    const int threads = n >= 256 ? 256 : ((n + 31) / 32) * 32;
    const dim3 grid(T, groups), block(threads);
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(gated_group_norm_kernel<bf16>, grid, block, 0, stream, o, (const bf16*)gate,
                              gate_stride, gain, (bf16*)out, width, groups, eps, gate_act, gate_first);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(gated_group_norm_kernel<float>, grid, block, 0, stream, o, (const float*)gate,
                              gate_stride, gain, (float*)out, width, groups, eps, gate_act, gate_first);
    return TGO_E_BAD_ARG;
}

// ---------------------------------------------------------------------------------------
// out = sa * a + sb * b, float32 (b null: out = sa * a; b may be `out` itself when it is
// float32, which accumulates). For the weighted sum of mixers that share an input.
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float sa, const T* b, float sb, float* out,
                                  long long n) {
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = b ? fmaf(sa, to_f32(a[i]), sb * to_f32(b[i])) : sa * to_f32(a[i]);
}

TGO_API int tgo_scaled_sum(const void* a, float sa, const void* b, float sb, float* out, int dtype,
                           long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256;
    const dim3 grid((unsigned)(want > 4096 ? 4096 : want));
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(scaled_sum_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)a, sa,
                              (const bf16*)b, sb, out, n);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(scaled_sum_kernel<float>, grid, dim3(256), 0, stream, (const float*)a, sa,
                              (const float*)b, sb, out, n);
    return TGO_E_BAD_ARG;
}

// -------------------------------- h <- gain * rmsnorm(alpha * h + y + bias)  (+ its copy)
// The arrangement with the norm AFTER the sum: the stream itself is what the norm leaves. A
// block a row: the sum s = alpha * h + y (+ bias, float32 [d], a product's bias that was left
// for here) is kept in shared memory in float32, divided by sqrt(mean s^2 + eps), multiplied
// by the gain and written back over h; `act`, if given, gets the same values in the
// activation type for the next sublayer to read.
template <typename TY, typename TA>
__global__ void scaled_add_norm_kernel(float* __restrict__ h, const TY* __restrict__ y,
                                       const float* __restrict__ bias, float alpha,
                                       const float* __restrict__ gain, float eps, int d,
                                       TA* __restrict__ act) {
    extern __shared__ float srow[];
    __shared__ float scratch[33];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float s = alpha * h[base + i] + to_f32(y[base + i]);
        if (bias) s += bias[i];
        srow[i] = s;
        ss += s * s;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = (srow[i] * r) * gain[i];
        h[base + i] = v;
        if (act) act[base + i] = from_f32<TA>(v);
    }
}

// h float32 [T, d] (in place); y [T, d] float32 or bfloat16; act bfloat16 [T, d] or null.
TGO_API int tgo_scaled_add_norm(float* h, const void* y, int y_dtype, const float* bias, float alpha,
                                const float* gain, float eps, void* act, int T, int d,
                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || (size_t)d * sizeof(float) > 200 * 1024) return TGO_E_BAD_ARG;
    const int threads = d >= 2048 ? 512 : d >= 512 ? 256 : 128;
    const size_t smem = (size_t)d * sizeof(float);
    if (y_dtype == TGO_F32) {
        auto kern = scaled_add_norm_kernel<float, bf16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, dim3(T), dim3(threads), smem, stream, h, (const float*)y, bias, alpha,
                              gain, eps, d, (bf16*)act);
    }
    if (y_dtype == TGO_BF16) {
        auto kern = scaled_add_norm_kernel<bf16, bf16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, dim3(T), dim3(threads), smem, stream, h, (const bf16*)y, bias, alpha,
                              gain, eps, d, (bf16*)act);
    }
    return TGO_E_BAD_ARG;
}

// ----------------------------------------------------------------- y += bias, row by row
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, int d, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = from_f32<T>(to_f32(y[i]) + bias[i % d]);
}

TGO_API int tgo_add_bias(void* y, int dtype, const float* bias, int T, int d, cudaStream_t stream) {
    if (T <= 0 || d <= 0) return 0;
    const size_t n = (size_t)T * d;
    const dim3 grid((unsigned)((n + 255) / 256)), block(256);
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(add_bias_kernel<bf16>, grid, block, 0, stream, (bf16*)y, bias, d, n);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(add_bias_kernel<float>, grid, block, 0, stream, (float*)y, bias, d, n);
    return TGO_E_BAD_ARG;
}

// ------------------------------------------------------------ several residual streams
// A layer arrangement that keeps S copies of the residual stream (x [S, T, d], float32) and
// learns how a sublayer reads them and writes back:
//   read    u = sum_s cin[s] x_s;  out = gain * rmsnorm(u)               (the sublayer's input)
//   write   x_t <- sum_s mix[s][t] x_s + cout[t] * y                      (all t from the old x)
// The write may also make the next sublayer's input from the new streams (next_in, next_gain:
// the row is kept in shared memory between the sum of squares and the output), and the plain
// sum of the new streams (sum_out). A block a token; everything float32 but y and out.
#define HC_MAX_STREAMS 8

__global__ void stream_spread_kernel(const float* __restrict__ h, float* __restrict__ x, size_t n,
                                     int S) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = h[i];
    for (int s = 0; s < S; ++s) x[(size_t)s * n + i] = v;
}

TGO_API int tgo_stream_spread(const float* h, float* x, long long n, int S, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (S <= 0 || S > HC_MAX_STREAMS) return TGO_E_BAD_ARG;
    return tgo_launch_pdl(stream_spread_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                          h, x, (size_t)n, S);
}

template <typename TO>
__global__ void __launch_bounds__(256)
stream_read_norm_kernel(const float* __restrict__ x, int S, int T, int d,
                        const float* __restrict__ cin, const float* __restrict__ gain, float eps,
                        TO* __restrict__ out) {
    extern __shared__ float row[];             // [d]
    __shared__ float scratch[33];
    pdl_wait();
    const size_t t = blockIdx.x, plane = (size_t)T * d;
    float c[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) c[s] = s < S ? cin[s] : 0.f;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) u = fmaf(c[s], x[s * plane + t * d + i], u);
        row[i] = u;
        ss += u * u;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[t * d + i] = from_f32<TO>((row[i] * r) * gain[i]);
}

// Four consecutive channels a thread and step (16-byte accesses of the float32 streams): for
// d % 4 == 0 and rows that start on 16 bytes. Same sums in the same order per channel; the sum of
// squares adds the four channels of a thread before the block's reduction.
__device__ __forceinline__ float4 hc_ld4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 hc_ld4(const bf16* p) {
    const uint2 r = *(const uint2*)p;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&r.x);
    const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)&r.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void hc_st4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void hc_st4(bf16* p, float4 v) {
    uint2 r;
    *(__nv_bfloat162*)&r.x = __floats2bfloat162_rn(v.x, v.y);
    *(__nv_bfloat162*)&r.y = __floats2bfloat162_rn(v.z, v.w);
    *(uint2*)p = r;
}

template <typename TO>
__global__ void __launch_bounds__(256)
stream_read_norm_vec_kernel(const float* __restrict__ x, int S, int T, int d,
                            const float* __restrict__ cin, const float* __restrict__ gain, float eps,
                            TO* __restrict__ out) {
    extern __shared__ float4 row4[];           // [d / 4]
    __shared__ float scratch[33];
    pdl_wait();
    const size_t t = blockIdx.x, plane = (size_t)T * d;
    float c[HC_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < HC_MAX_STREAMS; ++s) c[s] = s < S ? cin[s] : 0.f;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        float4 v[HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) v[s] = hc_ld4(x + s * plane + t * d + 4 * i);
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) {
                u.x = fmaf(c[s], v[s].x, u.x); u.y = fmaf(c[s], v[s].y, u.y);
                u.z = fmaf(c[s], v[s].z, u.z); u.w = fmaf(c[s], v[s].w, u.w);
            }
        row4[i] = u;
        ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        const float4 u = row4[i], g = *(const float4*)(gain + 4 * i);
        hc_st4(out + t * d + 4 * i, make_float4((u.x * r) * g.x, (u.y * r) * g.y, (u.z * r) * g.z, (u.w * r) * g.w));
    }
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
stream_write_vec_kernel(float* __restrict__ x, int S, int T, int d, const TY* __restrict__ y,
                        const float* __restrict__ mix, const float* __restrict__ cout,
                        const float* __restrict__ next_in, const float* __restrict__ next_gain, float eps,
                        TO* __restrict__ next_out, float* __restrict__ sum_out) {
    extern __shared__ float4 row4[];           // [d / 4] when the next input is made here
    __shared__ float scratch[33];
    __shared__ float m[HC_MAX_STREAMS * HC_MAX_STREAMS], co[HC_MAX_STREAMS], ni[HC_MAX_STREAMS];
    pdl_wait();
    if (threadIdx.x < S * S) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        co[threadIdx.x] = cout[threadIdx.x];
        ni[threadIdx.x] = next_in ? next_in[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const size_t t = blockIdx.x, plane = (size_t)T * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        float4 old[HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) old[s] = hc_ld4(x + s * plane + t * d + 4 * i);
        const float4 yv = hc_ld4(y + t * d + 4 * i);
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f), total = u;
#pragma unroll
        for (int to = 0; to < HC_MAX_STREAMS; ++to) {
            if (to >= S) continue;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) {
                    const float w = m[s * S + to];
                    a.x = fmaf(w, old[s].x, a.x); a.y = fmaf(w, old[s].y, a.y);
                    a.z = fmaf(w, old[s].z, a.z); a.w = fmaf(w, old[s].w, a.w);
                }
            a.x = fmaf(co[to], yv.x, a.x); a.y = fmaf(co[to], yv.y, a.y);
            a.z = fmaf(co[to], yv.z, a.z); a.w = fmaf(co[to], yv.w, a.w);
            hc_st4(x + to * plane + t * d + 4 * i, a);
            u.x = fmaf(ni[to], a.x, u.x); u.y = fmaf(ni[to], a.y, u.y);
            u.z = fmaf(ni[to], a.z, u.z); u.w = fmaf(ni[to], a.w, u.w);
            total.x += a.x; total.y += a.y; total.z += a.z; total.w += a.w;
        }
        if (sum_out) hc_st4(sum_out + t * d + 4 * i, total);
        if (next_out) {
            row4[i] = u;
            ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
        }
    }
    if (!next_out) return;
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        const float4 u = row4[i], g = *(const float4*)(next_gain + 4 * i);
        hc_st4(next_out + t * d + 4 * i, make_float4((u.x * r) * g.x, (u.y * r) * g.y, (u.z * r) * g.z, (u.w * r) * g.w));
    }
}

TGO_API int tgo_stream_read_norm(const float* x, int S, int T, int d, const float* cin,
                                 const float* gain, float eps, void* out, int out_dtype,
                                 cudaStream_t stream) {
    if (T <= 0) return 0;
    if (S <= 0 || S > HC_MAX_STREAMS || d <= 0 || d > 24576) return TGO_E_BAD_ARG;
    const size_t smem = (size_t)d * sizeof(float);
    const bool vec = d % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)gain & 15) && !((uintptr_t)out & 15);
    if (vec && out_dtype == TGO_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(stream_read_norm_vec_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(stream_read_norm_vec_kernel<bf16>, dim3(T), dim3(256), smem, stream, x, S, T, d,
                              cin, gain, eps, (bf16*)out);
    }
    if (vec && out_dtype == TGO_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(stream_read_norm_vec_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(stream_read_norm_vec_kernel<float>, dim3(T), dim3(256), smem, stream, x, S, T, d,
                              cin, gain, eps, (float*)out);
    }
    if (out_dtype == TGO_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(stream_read_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(stream_read_norm_kernel<bf16>, dim3(T), dim3(256), smem, stream, x, S, T, d,
                              cin, gain, eps, (bf16*)out);
    }
    if (out_dtype != TGO_F32) return TGO_E_BAD_ARG;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(stream_read_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return tgo_launch_pdl(stream_read_norm_kernel<float>, dim3(T), dim3(256), smem, stream, x, S, T, d, cin,
                          gain, eps, (float*)out);
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
stream_write_kernel(float* __restrict__ x, int S, int T, int d, const TY* __restrict__ y,
                    const float* __restrict__ mix, const float* __restrict__ cout,
                    const float* __restrict__ next_in, const float* __restrict__ next_gain, float eps,
                    TO* __restrict__ next_out, float* __restrict__ sum_out) {
    extern __shared__ float row[];             // [d] when the next input is made here
    __shared__ float scratch[33];
    __shared__ float m[HC_MAX_STREAMS * HC_MAX_STREAMS], co[HC_MAX_STREAMS], ni[HC_MAX_STREAMS];
    pdl_wait();
    if (threadIdx.x < S * S) m[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        co[threadIdx.x] = cout[threadIdx.x];
        ni[threadIdx.x] = next_in ? next_in[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const size_t t = blockIdx.x, plane = (size_t)T * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float old[HC_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HC_MAX_STREAMS; ++s)
            if (s < S) old[s] = x[s * plane + t * d + i];
        const float yv = to_f32(y[t * d + i]);
        float u = 0.f, total = 0.f;
#pragma unroll
        for (int to = 0; to < HC_MAX_STREAMS; ++to) {
            if (to >= S) continue;
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) a = fmaf(m[s * S + to], old[s], a);
            a = fmaf(co[to], yv, a);
            x[to * plane + t * d + i] = a;
            u = fmaf(ni[to], a, u);
            total += a;
        }
        if (sum_out) sum_out[t * d + i] = total;
        if (next_out) {
            row[i] = u;
            ss += u * u;
        }
    }
    if (!next_out) return;
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        next_out[t * d + i] = from_f32<TO>((row[i] * r) * next_gain[i]);
}

// y [T, d] in y_dtype; next_out [T, d] in out_dtype (with next_in [S], next_gain [d]) or null;
// sum_out float32 [T, d] or null.
TGO_API int tgo_stream_write(float* x, int S, int T, int d, const void* y, int y_dtype,
                             const float* mix, const float* cout, const float* next_in,
                             const float* next_gain, float eps, void* next_out, int out_dtype,
                             float* sum_out, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (S <= 0 || S > HC_MAX_STREAMS || d <= 0 || d > 24576) return TGO_E_BAD_ARG;
    if (next_out && (!next_in || !next_gain)) return TGO_E_BAD_ARG;
    const size_t smem = next_out ? (size_t)d * sizeof(float) : 0;
#define HC_GO(TY, TO)                                                                              \
    do {                                                                                           \
        if (smem > 48 * 1024)                                                                      \
            cudaFuncSetAttribute(stream_write_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tgo_launch_pdl(stream_write_kernel<TY, TO>, dim3(T), dim3(256), smem, stream, x, S, T, d, \
                              (const TY*)y, mix, cout, next_in, next_gain, eps, (TO*)next_out, sum_out); \
    } while (0)
#define HC_GO4(TY, TO)                                                                             \
    do {                                                                                           \
        if (smem > 48 * 1024)                                                                      \
            cudaFuncSetAttribute(stream_write_vec_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tgo_launch_pdl(stream_write_vec_kernel<TY, TO>, dim3(T), dim3(256), smem, stream, x, S, T, d, \
                              (const TY*)y, mix, cout, next_in, next_gain, eps, (TO*)next_out, sum_out); \
    } while (0)
    const bool out_bf = next_out && out_dtype == TGO_BF16;
    if (next_out && out_dtype != TGO_BF16 && out_dtype != TGO_F32) return TGO_E_BAD_ARG;
    const bool vec = d % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)y & 15) && !((uintptr_t)next_gain & 15) &&
                     !((uintptr_t)next_out & 15) && !((uintptr_t)sum_out & 15);
    if (vec && y_dtype == TGO_BF16) { if (out_bf) HC_GO4(bf16, bf16); else HC_GO4(bf16, float); }
    if (vec && y_dtype == TGO_F32) { if (out_bf) HC_GO4(float, bf16); else HC_GO4(float, float); }
    if (y_dtype == TGO_BF16) { if (out_bf) HC_GO(bf16, bf16); else HC_GO(bf16, float); }
    if (y_dtype == TGO_F32) { if (out_bf) HC_GO(float, bf16); else HC_GO(float, float); }
#undef HC_GO4
#undef HC_GO
    return TGO_E_BAD_ARG;
}

// ---------------------------------------------------------------- an activation in place
// x <- act(x) over [T, f] rows: the hidden rows of a feed-forward without a gate. Codes as in
// gated_act, and 3: the square of relu.
template <typename T>
__global__ void act_rows_kernel(T* __restrict__ x, size_t n, int act) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = to_f32(x[i]);
    float a;
    if (act == 1) a = z > 0.f ? z : 0.f;
    else if (act == 2) a = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    else if (act == 3) a = z > 0.f ? z * z : 0.f;
    else a = z / (1.f + expf(-z));
    x[i] = from_f32<T>(a);
}

TGO_API int tgo_act_rows(void* x, int dtype, long long n, int act, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (act < 0 || act > 3) return TGO_E_BAD_ARG;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(act_rows_kernel<bf16>, grid, dim3(256), 0, stream, (bf16*)x, (size_t)n, act);
    if (dtype == TGO_F32)
        return tgo_launch_pdl(act_rows_kernel<float>, grid, dim3(256), 0, stream, (float*)x, (size_t)n, act);
    return TGO_E_BAD_ARG;
}
