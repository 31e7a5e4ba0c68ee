// Matrix memory with exponential gates (the mLSTM of xLSTM). Per request and head a float32
// state is carried from token to token: a matrix S [dk][dv], a vector n [dk] and a running
// maximum m (all zero when a request starts; m starts at 0, not at minus infinity):
//
//   m_t = max(f_t + m_(t-1), i_t)
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// with the log gates i_t = cap tanh((a_t + b_i) / cap), f_t = logsigmoid(cap tanh((c_t + b_f) /
// cap)) made here, in float32, from the gate projections' raw rows a, c (float32). q is
// multiplied by q_scale as it is read. A step's tokens of one request are taken in chunks of up
// to ML_CHUNK tokens; with F_t the sum of f over the chunk's tokens up to t and m_0, S_0, n_0
// what the chunk starts from, the recurrence written out is
//
//   m_t = max(F_t + m_0, max_{s<=t} (F_t - F_s + i_s))
//   S_t = exp(F_t + m_0 - m_t) S_0 + sum_{s<=t} exp(F_t - F_s + i_s - m_t) k_s v_s^T
//
// in which no exponent is positive. Two kernels: the first, a block per (request, head), walks
// the gates, m, n and the denominators and leaves (f, i, m, denominator) per token and head in
// scratch, and the new n and m in the state; the second, a block per (request, head, slice of
// dv columns), keeps its slice of S in shared memory and makes the outputs. The second reads
// the m a request started from out of scratch, since the first has overwritten the state's.
//
// State row of a request: S [H][dk][dv], then n [H][dk], then m [H], float32.
#include "common.cuh"

#define ML_CHUNK 32
#define ML_THREADS 256

__device__ __forceinline__ float ml_log_sigmoid(float x) {
    // log(1 / (1 + exp(-x))) without overflow on either side
    return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
}

// The chunk's cumulative forget sums and running maxima, by one thread in token order:
// F[t] (inclusive), M[t]; M0 is the maximum the chunk starts from.
__device__ __forceinline__ void ml_walk(const float* lf, const float* li, int n, float M0, float* F,
                                        float* M) {
    float f = 0.f, m = M0;
    for (int t = 0; t < n; ++t) {
        f += lf[t];
        m = fmaxf(lf[t] + m, li[t]);
        F[t] = f;
        M[t] = m;
    }
}

template <typename T>
__global__ void __launch_bounds__(ML_THREADS)
mlstm_gates_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                   long long k_stride, const float* __restrict__ gi_raw, const float* __restrict__ gf_raw,
                   long long g_stride, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                   float cap, float q_scale, int H, int dk, int dv, const int* __restrict__ q_start,
                   const int* __restrict__ state_slots, float* __restrict__ state, long long state_row,
                   float* __restrict__ rec, float* __restrict__ m_first) {
    extern __shared__ float smem[];
    const int dkp = dk + 1;
    float* Qs = smem;                               // [ML_CHUNK][dk + 1]
    float* Ks = Qs + ML_CHUNK * dkp;                // [ML_CHUNK][dk + 1]
    float* As = Ks + ML_CHUNK * dkp;                // [ML_CHUNK][ML_CHUNK + 1]
    float* ns = As + ML_CHUNK * (ML_CHUNK + 1);     // [dk]
    float* lf = ns + dk;                            // [ML_CHUNK] each: log forget, log input,
    float* li = lf + ML_CHUNK;                      // cumulative forget, running maximum
    float* F = li + ML_CHUNK;
    float* M = F + ML_CHUNK;
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (t1 <= t0) return;
    float* row = state + (size_t)state_slots[b] * state_row;
    float* n_g = row + (size_t)H * dk * dv + (size_t)h * dk;
    float* m_g = row + (size_t)H * dk * dv + (size_t)H * dk + h;
    for (int d = threadIdx.x; d < dk; d += ML_THREADS) ns[d] = n_g[d];
    float m0 = *m_g;
    if (threadIdx.x == 0) m_first[(size_t)b * H + h] = m0;
    for (int ts = t0; ts < t1; ts += ML_CHUNK) {
        const int n = (t1 - ts) < ML_CHUNK ? (t1 - ts) : ML_CHUNK;
        __syncthreads();
        for (int i = threadIdx.x; i < n * dk; i += ML_THREADS) {
            const int r = i / dk, d = i % dk;
            const size_t t = (size_t)(ts + r);
            Qs[r * dkp + d] = to_f32(q[t * q_stride + (size_t)h * dk + d]) * q_scale;
            Ks[r * dkp + d] = to_f32(k[t * k_stride + (size_t)h * dk + d]);
        }
        if (threadIdx.x < n) {
            const size_t t = (size_t)(ts + threadIdx.x);
            const float a = gi_raw[t * g_stride + h] + bias_i[h];
            const float c = gf_raw[t * g_stride + h] + bias_f[h];
            li[threadIdx.x] = cap * tanhf(a / cap);
            lf[threadIdx.x] = ml_log_sigmoid(cap * tanhf(c / cap));
        }
        __syncthreads();
        if (threadIdx.x == 0) ml_walk(lf, li, n, m0, F, M);
        __syncthreads();
        // A[t][s] = (q_t . k_s) exp(F_t - F_s + i_s - m_t) for s <= t
        for (int idx = threadIdx.x; idx < n * n; idx += ML_THREADS) {
            const int i = idx / n, j = idx % n;
            float a = 0.f;
            if (j <= i) {
                const float* qi = Qs + i * dkp;
                const float* kj = Ks + j * dkp;
                for (int d = 0; d < dk; ++d) a += qi[d] * kj[d];
                a *= expf(F[i] - F[j] + li[j] - M[i]);
            }
            As[i * (ML_CHUNK + 1) + j] = a;
        }
        __syncthreads();
        // n_t . q_t and the denominator; a warp a token
        for (int i = threadIdx.x >> 5; i < n; i += ML_THREADS / 32) {
            const int lane = threadIdx.x & 31;
            float far = 0.f;
            for (int d = lane; d < dk; d += 32) far += ns[d] * Qs[i * dkp + d];
            far = warp_sum(far);
            float near = lane <= i ? As[i * (ML_CHUNK + 1) + lane] : 0.f;
            near = warp_sum(near);
            if (lane == 0) {
                const float nq = expf(F[i] + m0 - M[i]) * far + near;
                float* r = rec + ((size_t)(ts + i) * H + h) * 4;
                r[0] = lf[i];
                r[1] = li[i];
                r[2] = M[i];
                r[3] = fmaxf(fabsf(nq), expf(-M[i])) + 1e-6f;
            }
        }
        __syncthreads();
        const float keep = expf(F[n - 1] + m0 - M[n - 1]);
        for (int d = threadIdx.x; d < dk; d += ML_THREADS) {
            float a = 0.f;
            for (int j = 0; j < n; ++j) a += expf(F[n - 1] - F[j] + li[j] - M[n - 1]) * Ks[j * dkp + d];
            ns[d] = keep * ns[d] + a;
        }
        m0 = M[n - 1];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < dk; d += ML_THREADS) n_g[d] = ns[d];
    if (threadIdx.x == 0) *m_g = m0;
}

template <typename T>
__global__ void __launch_bounds__(ML_THREADS)
mlstm_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k, long long k_stride,
             const T* __restrict__ v, long long v_stride, float* __restrict__ out, float q_scale, int H,
             int dk, int dv, int vs, const int* __restrict__ q_start, const int* __restrict__ state_slots,
             float* __restrict__ state, long long state_row, const float* __restrict__ rec,
             const float* __restrict__ m_first) {
    extern __shared__ float smem[];
    const int dkp = dk + 1;
    float* Qs = smem;                               // [ML_CHUNK][dk + 1]
    float* Ks = Qs + ML_CHUNK * dkp;                // [ML_CHUNK][dk + 1]
    float* Vs = Ks + ML_CHUNK * dkp;                // [ML_CHUNK][vs]
    float* As = Vs + ML_CHUNK * vs;                 // [ML_CHUNK][ML_CHUNK + 1]
    float* Ss = As + ML_CHUNK * (ML_CHUNK + 1);     // [dk][vs]
    float* lf = Ss + (size_t)dk * vs;               // [ML_CHUNK] each
    float* li = lf + ML_CHUNK;
    float* M = li + ML_CHUNK;
    float* den = M + ML_CHUNK;
    float* F = den + ML_CHUNK;
    float* wk = F + ML_CHUNK;                       // weight of token s in the chunk's last state
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int c0 = blockIdx.z * vs;
    const int nc = (dv - c0) < vs ? (dv - c0) : vs;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (t1 <= t0) return;
    float* Sg = state + (size_t)state_slots[b] * state_row + ((size_t)h * dk) * dv + c0;
    for (int i = threadIdx.x; i < dk * vs; i += ML_THREADS) {
        const int d = i / vs, c = i % vs;
        Ss[i] = c < nc ? Sg[(size_t)d * dv + c] : 0.f;
    }
    float m0 = m_first[(size_t)b * H + h];
    for (int ts = t0; ts < t1; ts += ML_CHUNK) {
        const int n = (t1 - ts) < ML_CHUNK ? (t1 - ts) : ML_CHUNK;
        __syncthreads();
        for (int i = threadIdx.x; i < n * dk; i += ML_THREADS) {
            const int r = i / dk, d = i % dk;
            const size_t t = (size_t)(ts + r);
            Qs[r * dkp + d] = to_f32(q[t * q_stride + (size_t)h * dk + d]) * q_scale;
            Ks[r * dkp + d] = to_f32(k[t * k_stride + (size_t)h * dk + d]);
        }
        for (int i = threadIdx.x; i < n * vs; i += ML_THREADS) {
            const int r = i / vs, c = i % vs;
            Vs[i] = c < nc ? to_f32(v[(size_t)(ts + r) * v_stride + (size_t)h * dv + c0 + c]) : 0.f;
        }
        if (threadIdx.x < n) {
            const float* r = rec + ((size_t)(ts + threadIdx.x) * H + h) * 4;
            lf[threadIdx.x] = r[0];
            li[threadIdx.x] = r[1];
            M[threadIdx.x] = r[2];
            den[threadIdx.x] = r[3];
        }
        __syncthreads();
        if (threadIdx.x == 0) {                     // the same sums, in the same order, as the
            float f = 0.f;                          // first kernel's
            for (int t = 0; t < n; ++t) {
                f += lf[t];
                F[t] = f;
            }
        }
        __syncthreads();
        if (threadIdx.x < n) wk[threadIdx.x] = expf(F[n - 1] - F[threadIdx.x] + li[threadIdx.x] - M[n - 1]);
        for (int idx = threadIdx.x; idx < n * n; idx += ML_THREADS) {
            const int i = idx / n, j = idx % n;
            float a = 0.f;
            if (j <= i) {
                const float* qi = Qs + i * dkp;
                const float* kj = Ks + j * dkp;
                for (int d = 0; d < dk; ++d) a += qi[d] * kj[d];
                a *= expf(F[i] - F[j] + li[j] - M[i]);
            }
            As[i * (ML_CHUNK + 1) + j] = a;
        }
        __syncthreads();
        // o_t[c] = (exp(F_t + m_0 - m_t) q_t . S_0[:, c] + sum_s A[t][s] v_s[c]) / den_t
        for (int idx = threadIdx.x; idx < n * vs; idx += ML_THREADS) {
            const int i = idx / vs, c = idx % vs;
            if (c >= nc) continue;
            const float* qi = Qs + i * dkp;
            float far = 0.f;
            for (int d = 0; d < dk; ++d) far += qi[d] * Ss[d * vs + c];
            float near = 0.f;
            const float* ai = As + i * (ML_CHUNK + 1);
            for (int j = 0; j <= i; ++j) near += ai[j] * Vs[j * vs + c];
            out[((size_t)(ts + i) * H + h) * dv + c0 + c] = (expf(F[i] + m0 - M[i]) * far + near) / den[i];
        }
        __syncthreads();
        const float keep = expf(F[n - 1] + m0 - M[n - 1]);
        for (int idx = threadIdx.x; idx < dk * vs; idx += ML_THREADS) {
            const int d = idx / vs, c = idx % vs;
            float a = 0.f;
            for (int j = 0; j < n; ++j) a += wk[j] * Ks[j * dkp + d] * Vs[j * vs + c];
            Ss[idx] = keep * Ss[idx] + a;
        }
        m0 = M[n - 1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < dk * vs; i += ML_THREADS) {
        const int d = i / vs, c = i % vs;
        if (c < nc) Sg[(size_t)d * dv + c] = Ss[i];
    }
}

static inline size_t mlstm_gates_smem(int dk) {
    return ((size_t)2 * ML_CHUNK * (dk + 1) + (size_t)ML_CHUNK * (ML_CHUNK + 1) + dk + 4 * ML_CHUNK) *
           sizeof(float);
}
static inline size_t mlstm_smem(int dk, int vs) {
    return ((size_t)2 * ML_CHUNK * (dk + 1) + (size_t)ML_CHUNK * vs + (size_t)ML_CHUNK * (ML_CHUNK + 1) +
            (size_t)dk * vs + 6 * ML_CHUNK) * sizeof(float);
}

TGO_API long long tgo_mlstm_state_floats(int H, int dk, int dv) {
    return (long long)H * dk * dv + (long long)H * dk + H;
}

// q, k: [T, >= H*dk] rows (strided), v: [T, >= H*dv]; gi_raw, gf_raw float32 [T, >= H] with a
// common row stride; bias_i, bias_f float32 [H]; out float32 [T, H*dv]; state float32
// [slots, state_row]; rec float32 [T, H, 4] and m_first float32 [B, H] are scratch.
TGO_API int tgo_mlstm(const void* q, long long q_stride, const void* k, long long k_stride, const void* v,
                      long long v_stride, int dtype, const float* gi_raw, const float* gf_raw,
                      long long g_stride, const float* bias_i, const float* bias_f, float cap,
                      float q_scale, float* out, int B, int H, int dk, int dv, const int* q_start,
                      const int* state_slots, float* state, long long state_row, float* rec,
                      float* m_first, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || !(cap > 0.f) || !rec || !m_first ||
        state_row < tgo_mlstm_state_floats(H, dk, dv))
        return TGO_E_BAD_ARG;
    int vs = 32;                                    // columns of S a block owns
    while (vs > 8 && mlstm_smem(dk, vs) > 200 * 1024) vs >>= 1;
    const size_t smem = mlstm_smem(dk, vs), gsmem = mlstm_gates_smem(dk);
    if (smem > 200 * 1024 || gsmem > 200 * 1024) return TGO_E_BAD_ARG;
    const dim3 ggrid(B, H), grid(B, H, (dv + vs - 1) / vs), block(ML_THREADS);
    if (grid.z > 65535) return TGO_E_BAD_ARG;
    int rc;
#define ML_GO(TT)                                                                                          \
    {                                                                                                      \
        auto gk = mlstm_gates_kernel<TT>;                                                                  \
        auto mk = mlstm_kernel<TT>;                                                                        \
        if (gsmem > 48 * 1024) cudaFuncSetAttribute(gk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gsmem); \
        if (smem > 48 * 1024) cudaFuncSetAttribute(mk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        rc = tgo_launch_pdl(gk, ggrid, block, gsmem, stream, (const TT*)q, q_stride, (const TT*)k, k_stride, \
                            gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, q_scale, H, dk, dv, q_start,    \
                            state_slots, state, state_row, rec, m_first);                                  \
        if (rc) return rc;                                                                                 \
        return tgo_launch_pdl(mk, grid, block, smem, stream, (const TT*)q, q_stride, (const TT*)k, k_stride, \
                              (const TT*)v, v_stride, out, q_scale, H, dk, dv, vs, q_start, state_slots,   \
                              state, state_row, (const float*)rec, (const float*)m_first);                 \
    }
    if (dtype == TGO_BF16) ML_GO(bf16)
    if (dtype == TGO_F32) ML_GO(float)
#undef ML_GO
    return TGO_E_BAD_ARG;
}
