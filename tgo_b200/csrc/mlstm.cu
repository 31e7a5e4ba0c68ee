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

// ------------------------------------------------------------------ a step of single tokens
// One token a request. With m' = max(f + m, i), keep = exp(f + m - m'), take = exp(i - m'):
//
//   S <- keep S + take k v^T,   o = (keep S^T q + take (q . k) v) / (max(|keep n.q + take q.k|, exp(-m')) + 1e-6)
//
// straight from and to global memory, a block per (request, head, 32 columns of S), every
// element of S read once and written once. Every block of a (request, head) reads the old n
// and m; a second, small kernel writes the new ones afterwards.
#define MD_THREADS 128

__device__ __forceinline__ void ml_token_gates(const float* gi_raw, const float* gf_raw, long long g_stride,
                                               const float* bias_i, const float* bias_f, float cap, size_t t,
                                               int h, float m_old, float& m_new, float& keep, float& take) {
    const float li = cap * tanhf((gi_raw[t * g_stride + h] + bias_i[h]) / cap);
    const float lf = ml_log_sigmoid(cap * tanhf((gf_raw[t * g_stride + h] + bias_f[h]) / cap));
    m_new = fmaxf(lf + m_old, li);
    keep = expf(lf + m_old - m_new);
    take = expf(li - m_new);
}

template <typename T>
__global__ void __launch_bounds__(MD_THREADS)
mlstm_decode_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k, long long k_stride,
                    const T* __restrict__ v, long long v_stride, const float* __restrict__ gi_raw,
                    const float* __restrict__ gf_raw, long long g_stride, const float* __restrict__ bias_i,
                    const float* __restrict__ bias_f, float cap, float q_scale, float* __restrict__ out, int H,
                    int dk, int dv, const int* __restrict__ state_slots, float* __restrict__ state,
                    long long state_row) {
    extern __shared__ float smem[];
    float* qs = smem;                 // [dk]
    float* ks = qs + dk;              // [dk]
    float* red = ks + dk;             // [MD_THREADS / 32][32]
    __shared__ float part[2][MD_THREADS / 32];
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
    const int c = blockIdx.z * 32 + lane;
    const size_t t = (size_t)b;
    float* row = state + (size_t)state_slots[b] * state_row;
    const float* n_g = row + (size_t)H * dk * dv + (size_t)h * dk;
    const float m_old = row[(size_t)H * dk * dv + (size_t)H * dk + h];
    float qk = 0.f, nq = 0.f;
    for (int d = threadIdx.x; d < dk; d += MD_THREADS) {
        const float qq = to_f32(q[t * q_stride + (size_t)h * dk + d]) * q_scale;
        const float kk = to_f32(k[t * k_stride + (size_t)h * dk + d]);
        qs[d] = qq;
        ks[d] = kk;
        qk += qq * kk;
        nq += qq * n_g[d];
    }
    qk = warp_sum(qk);
    nq = warp_sum(nq);
    if (lane == 0) { part[0][rg] = qk; part[1][rg] = nq; }
    __syncthreads();
    constexpr int RG = MD_THREADS / 32;
    qk = nq = 0.f;
#pragma unroll
    for (int x = 0; x < RG; ++x) { qk += part[0][x]; nq += part[1][x]; }
    float m_new, keep, take;
    ml_token_gates(gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, t, h, m_old, m_new, keep, take);
    const float den = fmaxf(fabsf(keep * nq + take * qk), expf(-m_new)) + 1e-6f;
    const float vc = c < dv ? to_f32(v[t * v_stride + (size_t)h * dv + c]) : 0.f;
    float* Sg = row + ((size_t)h * dk) * dv;
    float far = 0.f;
    // eight rows of the state a thread and turn, all their loads before the stores
    for (int d0 = rg; d0 < dk; d0 += RG * 8) {
        float sv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int d = d0 + u * RG;
            sv[u] = (d < dk && c < dv) ? Sg[(size_t)d * dv + c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int d = d0 + u * RG;
            if (d < dk && c < dv) {
                far += qs[d] * sv[u];
                Sg[(size_t)d * dv + c] = keep * sv[u] + take * ks[d] * vc;
            }
        }
    }
    red[rg * 32 + lane] = far;
    __syncthreads();
    if (rg == 0 && c < dv) {
        float f = 0.f;
#pragma unroll
        for (int x = 0; x < RG; ++x) f += red[x * 32 + lane];
        out[(t * H + h) * dv + c] = (keep * f + take * qk * vc) / den;
    }
}

// after it: n <- keep n + take k and m <- m', a block a request, a thread per element of n
template <typename T>
__global__ void mlstm_decode_nm_kernel(const T* __restrict__ k, long long k_stride,
                                       const float* __restrict__ gi_raw, const float* __restrict__ gf_raw,
                                       long long g_stride, const float* __restrict__ bias_i,
                                       const float* __restrict__ bias_f, float cap, int H, int dk, int dv,
                                       const int* __restrict__ state_slots, float* __restrict__ state,
                                       long long state_row) {
    pdl_wait();
    const int b = blockIdx.x;
    float* row = state + (size_t)state_slots[b] * state_row;
    float* n_g = row + (size_t)H * dk * dv;
    float* m_g = n_g + (size_t)H * dk;
    // every thread reads the old m of its head before any thread writes a new one
    for (int e0 = 0; e0 < H * dk; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        float m_new = 0.f, keep = 0.f, take = 0.f;
        const int h = e < H * dk ? e / dk : 0;
        if (e < H * dk) ml_token_gates(gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, (size_t)b, h, m_g[h], m_new, keep, take);
        __syncthreads();
        if (e < H * dk) {
            n_g[e] = keep * n_g[e] + take * to_f32(k[(size_t)b * k_stride + e]);
            // the last element of a head writes its m, once no thread of this turn needs the old one;
            // heads that straddle two turns are written by the later turn alone
            if (e % dk == dk - 1) m_g[h] = m_new;
        }
        __syncthreads();
    }
}

// --------------------------------------------------------------- prompt portions, by chunks
// The tokens of a step are cut into chunks of up to MC_CHUNK tokens of one request (a list the
// host makes: first token row and count of each chunk). With F_s the sum of f over a chunk's
// tokens up to s, n its count and a_s = F_n - F_s + i_s:
//
//   summaries   b_c = max_s a_s;  U_c = sum_s exp(a_s - b_c) k_s v_s^T,  u_c likewise with k_s
//   scan        per request and head, chunk after chunk: the state before the chunk (P_c, p_c, m)
//               replaces its summary; m' = max(F_n + m, b_c), S <- exp(F_n + m - m') S + exp(b_c - m') U_c
//   outputs     m_t by the recurrence from the m before the chunk; per token
//               o_t = (exp(F_t + m - m_t) P_c^T q_t + sum_{s<=t} exp(F_t - F_s + i_s - m_t) (q_t . k_s) v_s) / den_t
//
// A record of scratch per (chunk, head): [dk][dv] matrix, [dk] vector, then F_n, b_c, the m before
// the chunk and the m after it. The scan leaves S and n in the state and every request's last m in
// `m_last`; the outputs kernel, which reads no m from the state, stores those.
#define MC_CHUNK 64
#define MC_THREADS 256
#define MC_VS 64

__device__ __forceinline__ size_t mc_record(int dk, int dv) { return (size_t)dk * dv + dk + 4; }

// log gates of a chunk's tokens into li, lf (threads 0..n-1), then F by one thread
__device__ __forceinline__ void mc_gates(const float* gi_raw, const float* gf_raw, long long g_stride,
                                         const float* bias_i, const float* bias_f, float cap, int h, int tok0,
                                         int n, float* li, float* lf, float* F) {
    if (threadIdx.x < n) {
        const size_t t = (size_t)(tok0 + threadIdx.x);
        li[threadIdx.x] = cap * tanhf((gi_raw[t * g_stride + h] + bias_i[h]) / cap);
        lf[threadIdx.x] = ml_log_sigmoid(cap * tanhf((gf_raw[t * g_stride + h] + bias_f[h]) / cap));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float f = 0.f;
        for (int t = 0; t < n; ++t) { f += lf[t]; F[t] = f; }
    }
    __syncthreads();
}

template <typename T>
__device__ __forceinline__ void mc_load(float* dst, int ld, const T* __restrict__ x, long long stride, int h,
                                        int dk, int tok0, int n, float mul) {
    for (int i0 = threadIdx.x; i0 < n * dk; i0 += 4 * MC_THREADS) {
        float val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * MC_THREADS;
            if (i < n * dk) val[u] = to_f32(x[(size_t)(tok0 + i / dk) * stride + (size_t)h * dk + i % dk]) * mul;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * MC_THREADS;
            if (i < n * dk) dst[(i / dk) * ld + i % dk] = val[u];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(MC_THREADS)
mlstm_summaries_kernel(const T* __restrict__ k, long long k_stride, const T* __restrict__ v, long long v_stride,
                       const float* __restrict__ gi_raw, const float* __restrict__ gf_raw, long long g_stride,
                       const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, int H,
                       int dk, int dv, const int* __restrict__ chunk_tok0, const int* __restrict__ chunk_ntok,
                       float* __restrict__ U) {
    extern __shared__ float smem[];
    const int ldk = dk + 1;
    float* Ks = smem;                         // [MC_CHUNK][dk + 1], rows times exp(a_s - b_c)
    float* Vs = Ks + MC_CHUNK * ldk;          // [MC_CHUNK][MC_VS]
    float* li = Vs + MC_CHUNK * MC_VS;        // [MC_CHUNK] each
    float* lf = li + MC_CHUNK;
    float* F = lf + MC_CHUNK;
    float* wk = F + MC_CHUNK;
    __shared__ float top;
    pdl_wait();
    const int ci = blockIdx.x, h = blockIdx.y;
    const int tok0 = chunk_tok0[ci], n = chunk_ntok[ci];
    mc_load(Ks, ldk, k, k_stride, h, dk, tok0, n, 1.f);
    mc_gates(gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, h, tok0, n, li, lf, F);
    if (threadIdx.x == 0) {
        float b = -INFINITY;
        for (int s = 0; s < n; ++s) b = fmaxf(b, F[n - 1] - F[s] + li[s]);
        top = b;
    }
    __syncthreads();
    if (threadIdx.x < n) wk[threadIdx.x] = expf(F[n - 1] - F[threadIdx.x] + li[threadIdx.x] - top);
    __syncthreads();
    for (int i = threadIdx.x; i < n * dk; i += MC_THREADS) Ks[(i / dk) * ldk + i % dk] *= wk[i / dk];
    float* Uo = U + ((size_t)ci * H + h) * mc_record(dk, dv);
    __syncthreads();
    for (int d = threadIdx.x; d < dk; d += MC_THREADS) {
        float a = 0.f;
        for (int j = 0; j < n; ++j) a += Ks[j * ldk + d];
        Uo[(size_t)dk * dv + d] = a;
    }
    if (threadIdx.x == 0) {
        Uo[(size_t)dk * dv + dk] = F[n - 1];
        Uo[(size_t)dk * dv + dk + 1] = top;
    }
    for (int c0 = 0; c0 < dv; c0 += MC_VS) {
        const int nc = dv - c0 < MC_VS ? dv - c0 : MC_VS;
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < n * MC_VS; i += MC_THREADS) {
            const int r = i / MC_VS, c = i % MC_VS;
            Vs[i] = c < nc ? to_f32(v[(size_t)(tok0 + r) * v_stride + (size_t)h * dv + c0 + c]) : 0.f;
        }
        __syncthreads();
        const int tiles_c = MC_VS / 4, tiles_d = (dk + 3) / 4;
        for (int tile = threadIdx.x; tile < tiles_d * tiles_c; tile += MC_THREADS) {
            const int d0 = (tile / tiles_c) * 4, cc = (tile % tiles_c) * 4;
            float acc[4][4] = {};
            for (int j = 0; j < n; ++j) {
                const float4 vv = *(const float4*)(Vs + j * MC_VS + cc);
                float kk[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) kk[x] = d0 + x < dk ? Ks[j * ldk + d0 + x] : 0.f;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    acc[x][0] += kk[x] * vv.x; acc[x][1] += kk[x] * vv.y;
                    acc[x][2] += kk[x] * vv.z; acc[x][3] += kk[x] * vv.w;
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y)
                    if (d0 + x < dk && cc + y < nc) Uo[(size_t)(d0 + x) * dv + c0 + cc + y] = acc[x][y];
        }
    }
}

// grid (requests, heads, ceil((dk * dv + dk) / 256)): a thread an element of S or of n
__global__ void mlstm_scan_kernel(int H, int dk, int dv, const int* __restrict__ q_start,
                                  const int* __restrict__ state_slots, const int* __restrict__ chunk_first,
                                  float* __restrict__ U, float* __restrict__ state, long long state_row,
                                  float* __restrict__ m_last) {
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int n_tok = q_start[b + 1] - q_start[b];
    if (e >= dk * dv + dk || n_tok <= 0) return;
    const int chunks = (n_tok + MC_CHUNK - 1) / MC_CHUNK;
    float* row = state + (size_t)state_slots[b] * state_row;
    float* sp = e < dk * dv ? row + (size_t)h * dk * dv + e : row + (size_t)H * dk * dv + (size_t)h * dk + (e - dk * dv);
    float s = *sp;
    float m = row[(size_t)H * dk * dv + (size_t)H * dk + h];
    const size_t step = (size_t)H * mc_record(dk, dv);
    float* ub = U + ((size_t)chunk_first[b] * H + h) * mc_record(dk, dv);
    const size_t meta = (size_t)dk * dv + dk;
    for (int cb = 0; cb < chunks; cb += 8) {        // eight summaries loaded ahead of their use
        float u[8], fn[8], top[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const bool in = cb + x < chunks;
            u[x] = in ? ub[(size_t)(cb + x) * step + e] : 0.f;
            fn[x] = in ? ub[(size_t)(cb + x) * step + meta] : 0.f;
            top[x] = in ? ub[(size_t)(cb + x) * step + meta + 1] : 0.f;
        }
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            const int c = cb + x;
            if (c < chunks) {
                ub[(size_t)c * step + e] = s;
                const float m_new = fmaxf(fn[x] + m, top[x]);
                s = expf(fn[x] + m - m_new) * s + expf(top[x] - m_new) * u[x];
                if (e == 0) {
                    ub[(size_t)c * step + meta + 2] = m;
                    ub[(size_t)c * step + meta + 3] = m_new;
                }
                m = m_new;
            }
        }
    }
    *sp = s;
    if (e == 0) m_last[(size_t)b * H + h] = m;
}

template <typename T>
__global__ void __launch_bounds__(MC_THREADS)
mlstm_outputs_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k, long long k_stride,
                     const T* __restrict__ v, long long v_stride, const float* __restrict__ gi_raw,
                     const float* __restrict__ gf_raw, long long g_stride, const float* __restrict__ bias_i,
                     const float* __restrict__ bias_f, float cap, float q_scale, float* __restrict__ out, int B,
                     int H, int dk, int dv, const int* __restrict__ chunk_tok0,
                     const int* __restrict__ chunk_ntok, const float* __restrict__ P,
                     const int* __restrict__ state_slots, float* __restrict__ state, long long state_row,
                     const float* __restrict__ m_last) {
    extern __shared__ float smem[];
    const int ldk = dk + 1, lda = MC_CHUNK + 1;
    float* Qs = smem;                          // [MC_CHUNK][dk + 1]
    float* Ks = Qs + MC_CHUNK * ldk;           // [MC_CHUNK][dk + 1]
    float* As = Ks + MC_CHUNK * ldk;           // [MC_CHUNK][MC_CHUNK + 1]
    float* Vs = As + MC_CHUNK * lda;           // [MC_CHUNK][MC_VS]
    float* Ss = Vs + MC_CHUNK * MC_VS;         // [dk][MC_VS]
    float* li = Ss + (size_t)dk * MC_VS;       // [MC_CHUNK] each
    float* lf = li + MC_CHUNK;
    float* F = lf + MC_CHUNK;
    float* M = F + MC_CHUNK;
    float* far_w = M + MC_CHUNK;               // exp(F_t + m - m_t)
    float* den = far_w + MC_CHUNK;
    pdl_wait();
    const int ci = blockIdx.x, h = blockIdx.y;
    const int tok0 = chunk_tok0[ci], n = chunk_ntok[ci];
    if (ci == 0)                               // every request's m after this step, for this head
        for (int b = threadIdx.x; b < B; b += MC_THREADS)
            state[(size_t)state_slots[b] * state_row + (size_t)H * dk * dv + (size_t)H * dk + h] =
                m_last[(size_t)b * H + h];
    const float* Pc = P + ((size_t)ci * H + h) * mc_record(dk, dv);
    const float* pn = Pc + (size_t)dk * dv;
    const float m0 = pn[dk + 2];
    mc_load(Qs, ldk, q, q_stride, h, dk, tok0, n, q_scale);
    mc_load(Ks, ldk, k, k_stride, h, dk, tok0, n, 1.f);
    mc_gates(gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, h, tok0, n, li, lf, F);
    if (threadIdx.x == 0) {
        float m = m0;
        for (int t = 0; t < n; ++t) { m = fmaxf(lf[t] + m, li[t]); M[t] = m; }
    }
    __syncthreads();
    // A[i][j] = (q_i . k_j) exp(F_i - F_j + i_j - m_i) (j <= i), 4 x 4 tiles
    {
        const int tiles = MC_CHUNK / 4;
        for (int tile = threadIdx.x; tile < tiles * tiles; tile += MC_THREADS) {
            const int i0 = (tile / tiles) * 4, j0 = (tile % tiles) * 4;
            if (i0 >= n || j0 >= n) continue;
            float acc[4][4] = {};
            if (j0 <= i0 + 3) {
                for (int d = 0; d < dk; ++d) {
                    float qq[4], kk[4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        qq[x] = Qs[(i0 + x) * ldk + d];          // rows >= n: dropped below
                        kk[x] = Ks[(j0 + x) * ldk + d];
                    }
#pragma unroll
                    for (int x = 0; x < 4; ++x)
#pragma unroll
                        for (int y = 0; y < 4; ++y) acc[x][y] += qq[x] * kk[y];
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const int i = i0 + x, j = j0 + y;
                    As[i * lda + j] = (j <= i && i < n) ? acc[x][y] * expf(F[i] - F[j] + li[j] - M[i]) : 0.f;
                }
        }
    }
    __syncthreads();
    // the denominators; a warp a token
    for (int i = threadIdx.x >> 5; i < n; i += MC_THREADS / 32) {
        const int lane = threadIdx.x & 31;
        float far = 0.f, near = 0.f;
        for (int d = lane; d < dk; d += 32) far += pn[d] * Qs[i * ldk + d];
        for (int j = lane; j <= i; j += 32) near += As[i * lda + j];
        far = warp_sum(far);
        near = warp_sum(near);
        if (lane == 0) {
            const float w = expf(F[i] + m0 - M[i]);
            far_w[i] = w;
            den[i] = fmaxf(fabsf(w * far + near), expf(-M[i])) + 1e-6f;
        }
    }
    for (int c0 = 0; c0 < dv; c0 += MC_VS) {
        const int nc = dv - c0 < MC_VS ? dv - c0 : MC_VS;
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < n * MC_VS; i += MC_THREADS) {
            const int r = i / MC_VS, c = i % MC_VS;
            Vs[i] = c < nc ? to_f32(v[(size_t)(tok0 + r) * v_stride + (size_t)h * dv + c0 + c]) : 0.f;
        }
#pragma unroll 8
        for (int i = threadIdx.x; i < dk * MC_VS; i += MC_THREADS) {
            const int d = i / MC_VS, c = i % MC_VS;
            Ss[i] = c < nc ? Pc[(size_t)d * dv + c0 + c] : 0.f;
        }
        __syncthreads();
        const int tiles_c = MC_VS / 4, tiles_i = (n + 3) / 4;
        for (int tile = threadIdx.x; tile < tiles_i * tiles_c; tile += MC_THREADS) {
            const int i0 = (tile / tiles_c) * 4, cc = (tile % tiles_c) * 4;
            float near[4][4] = {}, far[4][4] = {};
            const int jmax = i0 + 3 < n - 1 ? i0 + 3 : n - 1;
            for (int j = 0; j <= jmax; ++j) {
                const float4 vv = *(const float4*)(Vs + j * MC_VS + cc);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float a = As[(i0 + x) * lda + j];        // rows >= n were zeroed
                    near[x][0] += a * vv.x; near[x][1] += a * vv.y; near[x][2] += a * vv.z; near[x][3] += a * vv.w;
                }
            }
            for (int d = 0; d < dk; ++d) {
                const float4 ss = *(const float4*)(Ss + d * MC_VS + cc);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float qq = Qs[(i0 + x) * ldk + d];
                    far[x][0] += qq * ss.x; far[x][1] += qq * ss.y; far[x][2] += qq * ss.z; far[x][3] += qq * ss.w;
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y)
                    if (i0 + x < n && cc + y < nc)
                        out[((size_t)(tok0 + i0 + x) * H + h) * dv + c0 + cc + y] =
                            (near[x][y] + far_w[i0 + x] * far[x][y]) / den[i0 + x];
        }
    }
}

static inline size_t mc_summaries_smem(int dk) {
    return ((size_t)MC_CHUNK * (dk + 1) + (size_t)MC_CHUNK * MC_VS + 4 * MC_CHUNK) * sizeof(float);
}
static inline size_t mc_outputs_smem(int dk) {
    return ((size_t)2 * MC_CHUNK * (dk + 1) + (size_t)MC_CHUNK * (MC_CHUNK + 1) + (size_t)MC_CHUNK * MC_VS +
            (size_t)dk * MC_VS + 6 * MC_CHUNK) * sizeof(float);
}

TGO_API int tgo_mlstm_chunk_tokens() { return MC_CHUNK; }

// 1 if the chunked kernels (and the single-token kernels) take these sizes.
TGO_API int tgo_mlstm_chunked_supports(int H, int dk, int dv) {
    return (H > 0 && H <= 65535 && dk > 0 && dv > 0 && mc_outputs_smem(dk) <= 200 * 1024) ? 1 : 0;
}

TGO_API long long tgo_mlstm_chunk_record_floats(int dk, int dv) { return (long long)dk * dv + dk + 4; }

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

template <typename T>
static int mlstm_chunked(const T* q, long long q_stride, const T* k, long long k_stride, const T* v,
                         long long v_stride, const float* gi_raw, const float* gf_raw, long long g_stride,
                         const float* bias_i, const float* bias_f, float cap, float q_scale, float* out, int B,
                         int H, int dk, int dv, const int* q_start, const int* state_slots, float* state,
                         long long state_row, int chunks, const int* chunk_tok0, const int* chunk_ntok,
                         const int* chunk_first, float* scratch, float* m_last, int single,
                         cudaStream_t stream) {
    if (single) {
        const size_t smem = ((size_t)2 * dk + MD_THREADS) * sizeof(float);
        int rc = tgo_launch_pdl(mlstm_decode_kernel<T>, dim3(B, H, (dv + 31) / 32), dim3(MD_THREADS), smem, stream,
                                q, q_stride, k, k_stride, v, v_stride, gi_raw, gf_raw, g_stride, bias_i, bias_f,
                                cap, q_scale, out, H, dk, dv, state_slots, state, state_row);
        if (rc) return rc;
        return tgo_launch_pdl(mlstm_decode_nm_kernel<T>, dim3(B), dim3(256), 0, stream, k, k_stride, gi_raw,
                              gf_raw, g_stride, bias_i, bias_f, cap, H, dk, dv, state_slots, state, state_row);
    }
    const size_t s1 = mc_summaries_smem(dk), s3 = mc_outputs_smem(dk);
    auto k1 = mlstm_summaries_kernel<T>;
    auto k3 = mlstm_outputs_kernel<T>;
    if (s1 > 48 * 1024) cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1);
    if (s3 > 48 * 1024) cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s3);
    int rc = tgo_launch_pdl(k1, dim3(chunks, H), dim3(MC_THREADS), s1, stream, k, k_stride, v, v_stride, gi_raw,
                            gf_raw, g_stride, bias_i, bias_f, cap, H, dk, dv, chunk_tok0, chunk_ntok, scratch);
    if (rc) return rc;
    rc = tgo_launch_pdl(mlstm_scan_kernel, dim3(B, H, (dk * dv + dk + 255) / 256), dim3(256), 0, stream, H, dk, dv,
                        q_start, state_slots, chunk_first, scratch, state, state_row, m_last);
    if (rc) return rc;
    return tgo_launch_pdl(k3, dim3(chunks, H), dim3(MC_THREADS), s3, stream, q, q_stride, k, k_stride, v, v_stride,
                          gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, q_scale, out, B, H, dk, dv, chunk_tok0,
                          chunk_ntok, (const float*)scratch, state_slots, state, state_row, (const float*)m_last);
}

// As tgo_mlstm, by chunks. chunk_tok0 / chunk_ntok: the chunks (at most tgo_mlstm_chunk_tokens()
// tokens of one request each, a request's chunks in order and next to each other); chunk_first
// [B]: index of each request's first chunk; scratch: float32 [chunks, H,
// tgo_mlstm_chunk_record_floats]; m_last: float32 [B, H]. single != 0: every request brings one
// token (no chunk lists or scratch needed).
TGO_API int tgo_mlstm_chunked(const void* q, long long q_stride, const void* k, long long k_stride,
                              const void* v, long long v_stride, int dtype, const float* gi_raw,
                              const float* gf_raw, long long g_stride, const float* bias_i, const float* bias_f,
                              float cap, float q_scale, float* out, int B, int H, int dk, int dv,
                              const int* q_start, const int* state_slots, float* state, long long state_row,
                              int chunks, const int* chunk_tok0, const int* chunk_ntok, const int* chunk_first,
                              float* scratch, float* m_last, int single, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (!tgo_mlstm_chunked_supports(H, dk, dv) || !(cap > 0.f) || state_row < tgo_mlstm_state_floats(H, dk, dv) ||
        (!single && (chunks <= 0 || !chunk_tok0 || !chunk_ntok || !chunk_first || !scratch || !m_last)))
        return TGO_E_BAD_ARG;
    if (dtype == TGO_BF16)
        return mlstm_chunked<bf16>((const bf16*)q, q_stride, (const bf16*)k, k_stride, (const bf16*)v, v_stride,
                                   gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, q_scale, out, B, H, dk, dv,
                                   q_start, state_slots, state, state_row, chunks, chunk_tok0, chunk_ntok,
                                   chunk_first, scratch, m_last, single, stream);
    if (dtype == TGO_F32)
        return mlstm_chunked<float>((const float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride,
                                    gi_raw, gf_raw, g_stride, bias_i, bias_f, cap, q_scale, out, B, H, dk, dv,
                                    q_start, state_slots, state, state_row, chunks, chunk_tok0, chunk_ntok,
                                    chunk_first, scratch, m_last, single, stream);
    return TGO_E_BAD_ARG;
}
