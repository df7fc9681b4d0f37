// Gated linear attention: linear attention whose state decays per KEY CHANNEL by a factor that depends on the token.
//
// Per head, with q_t, k_t of size dk, v_t of size dv and a decay a_t in (0, 1)^dk:
//     a_t = sigmoid(z_t)^(1 / tau),  z_t = (low-rank projection of the token) + bias
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          (S: [dk, dv], zero at the start of a sequence)
//     o_t = S_t^T (q_t * q_scale)
//     y_t = o_t / sqrt(mean(o_t^2) + eps) * w * silu(g_t)       (w: [dv], the same for every head)
// The state, the decays (through log sigmoid, so that no power of a small number is formed), the sums, the unit norm and
// the gate are 32-bit in every engine dtype; S lives in the engine's per-sequence state rows [slot, H, dk, dv].
//
// A row of `proj` holds a token's projections q [H, dk] | k [H, dk] | v [H, dv] | g [H, dv] as float32; a row of `z` the
// decay logits [H, dk] WITHOUT their bias.
//
// Two forms:
//   * gla_seq_kernel: one block per (sequence, head) walks its tokens one after another with S in shared memory
//     (a decode step, short portions).
//   * the chunked form for long portions, over chunks of GC tokens of all sequences and heads at once.  With
//     b_t = sum_(s <= t) log a_s inside the chunk (all exponents below are <= 0, so nothing can overflow):
//       1. U_c = sum_j (k_j * exp(b_n - b_j)) v_j^T,  D_c = exp(b_n)      what chunk c (n tokens) adds, and its decay
//       2. S_c = diag(D_c) S_(c-1) + U_c, chunk after chunk               (U_c is overwritten by the state BEFORE c)
//       3. o_t = S_(c-1)^T (q_t * exp(b_t)) + sum_(j <= t) (sum_i q_t[i] k_j[i] exp(b_t[i] - b_j[i])) v_j, norm, gate
//     These are the recurrence's own terms in another order; nothing is approximated.
#include "common.cuh"

#define GLA_THREADS 256
#define GC 16                       // tokens a chunk

__device__ __forceinline__ float gla_silu(float z) { return z / (1.0f + expf(-z)); }
// log(sigmoid(z)) = min(z, 0) - log(1 + exp(-|z|))
__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename TO>
__global__ void __launch_bounds__(GLA_THREADS)
gla_seq_kernel(const float *__restrict__ proj, int ld, const float *__restrict__ z, int ldz, const float *__restrict__ z_bias,
               const float *__restrict__ norm_w, TO *__restrict__ out, int ldo, const int *__restrict__ cu_rows,
               const int *__restrict__ slots, float *__restrict__ state, int H, int dk, int dv, float inv_tau, float q_scale,
               float eps) {
    extern __shared__ float sm[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = cu_rows[seq], row1 = cu_rows[seq + 1];
    if (row1 <= row0) return;
    const int G = GLA_THREADS / dv, n_active = G * dv;      // threads (g, j): column j of S, rows g, g + G, ...
    float *S = sm, *qs = S + dk * dv, *ks = qs + dk, *as = ks + dk, *vs = as + dk, *part = vs + dv;
    float *Sg = state + ((size_t)slots[seq] * H + h) * dk * dv;
    for (int e = tid; e < dk * dv; e += GLA_THREADS) S[e] = Sg[e];
    for (int r = row0; r < row1; r++) {
        const float *row = proj + (size_t)r * ld;
        for (int i = tid; i < dk; i += GLA_THREADS) {
            qs[i] = row[(size_t)h * dk + i] * q_scale;
            ks[i] = row[(size_t)(H + h) * dk + i];
            as[i] = expf(log_sigmoid(z[(size_t)r * ldz + (size_t)h * dk + i] + z_bias[(size_t)h * dk + i]) * inv_tau);
        }
        for (int j = tid; j < dv; j += GLA_THREADS) vs[j] = row[(size_t)2 * H * dk + (size_t)h * dv + j];
        __syncthreads();
        if (tid < n_active) {
            const int j = tid % dv, g = tid / dv;
            const float vj = vs[j];
            float acc = 0.f;
            for (int i = g; i < dk; i += G) {
                float s = fmaf(S[i * dv + j], as[i], ks[i] * vj);
                S[i * dv + j] = s;
                acc = fmaf(s, qs[i], acc);
            }
            part[g * dv + j] = acc;
        }
        __syncthreads();
        float o = 0.f;
        if (tid < dv)
            for (int g = 0; g < G; g++) o += part[g * dv + tid];
        float ss = block_sum(tid < dv ? o * o : 0.f, scratch);
        if (tid < dv) {
            float gate = row[(size_t)2 * H * dk + (size_t)(H + h) * dv + tid];
            out[(size_t)r * ldo + (size_t)h * dv + tid] = from_f32<TO>(o * (1.0f / sqrtf(ss / (float)dv + eps)) * norm_w[tid] * gla_silu(gate));
        }
    }
    __syncthreads();
    for (int e = tid; e < dk * dv; e += GLA_THREADS) Sg[e] = S[e];
}

// ------------------------------------------------------------------ chunked form
// Chunk c covers tokens [chunk_row[c], chunk_row[c] + chunk_len[c]); the chunks of a sequence are consecutive and in order,
// sequence s owning chunks [seq_chunk0[s], seq_chunk0[s + 1]).  The plan is made on the device from the step's row offsets.
__global__ void gla_chunk_plan_kernel(const int *__restrict__ cu_rows, int n_seq, int *__restrict__ chunk_row, int *__restrict__ chunk_len,
                                      int *__restrict__ seq_chunk0) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int s = 0; s < n_seq; s++) { seq_chunk0[s] = at; at += (cu_rows[s + 1] - cu_rows[s] + GC - 1) / GC; }
        seq_chunk0[n_seq] = at;
    }
    __syncthreads();
    for (int s = threadIdx.x; s < n_seq; s += blockDim.x) {
        const int r0 = cu_rows[s], r1 = cu_rows[s + 1];
        int c = seq_chunk0[s];
        for (int r = r0; r < r1; r += GC, c++) { chunk_row[c] = r; chunk_len[c] = min(GC, r1 - r); }
    }
}

// b[t][i] = sum_(s <= t) log a_s[i] for the chunk's tokens, into shared memory (row stride dk): the logarithms of all
// (token, channel) pairs at once, a warp a token, then a running sum per channel.  Contains two __syncthreads().
__device__ __forceinline__ void gla_cumulative_log_decay(const float *__restrict__ z, int ldz, const float *__restrict__ z_bias, int r0, int n,
                                                         int h, int dk, float inv_tau, float *b, int tid) {
    for (int t = tid >> 5; t < n; t += GLA_THREADS / 32)
        for (int i = tid & 31; i < dk; i += 32)
            b[t * dk + i] = log_sigmoid(z[(size_t)(r0 + t) * ldz + (size_t)h * dk + i] + z_bias[(size_t)h * dk + i]) * inv_tau;
    __syncthreads();
    for (int i = tid; i < dk; i += GLA_THREADS) {
        float run = 0.f;
        for (int t = 0; t < n; t++) {
            run += b[t * dk + i];
            b[t * dk + i] = run;
        }
    }
    __syncthreads();
}

// 1. U[c, h] = sum_j (k_j * exp(b_n - b_j)) v_j^T and D[c, h] = exp(b_n).  One block per (chunk, head); thread (g, j) owns
// column j of U and rows g, g + G, ...: the chunk's values of column j wait in registers, the decayed keys of a row are read
// from shared memory as four 16-byte broadcasts.
__global__ void __launch_bounds__(GLA_THREADS)
gla_chunk_state_kernel(const float *__restrict__ proj, int ld, const float *__restrict__ z, int ldz, const float *__restrict__ z_bias,
                       const int *__restrict__ chunk_row, const int *__restrict__ chunk_len, float *__restrict__ U, float *__restrict__ D,
                       float *__restrict__ Bg, int H, int dk, int dv, float inv_tau) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int r0 = chunk_row[c], n = chunk_len[c];
    float *b = sm, *kd = b + GC * dk;                          // b: [GC][dk]; kd: [dk][GC], zero beyond the chunk's n tokens
    gla_cumulative_log_decay(z, ldz, z_bias, r0, n, h, dk, inv_tau, b, tid);
    // the outputs kernel reads the cumulative decays instead of forming them again
    for (int e = tid; e < n * dk; e += GLA_THREADS) Bg[((size_t)c * H + h) * GC * dk + e] = b[e];
    // (loops over a [token][channel] tile walk tokens by warp and channels by lane: no division by a run-time size)
    for (int t = tid >> 5; t < GC; t += GLA_THREADS / 32)
        for (int i = tid & 31; i < dk; i += 32)
            kd[i * GC + t] = t < n ? proj[(size_t)(r0 + t) * ld + (size_t)(H + h) * dk + i] * __expf(b[(n - 1) * dk + i] - b[t * dk + i]) : 0.f;
    for (int i = tid; i < dk; i += GLA_THREADS) D[((size_t)c * H + h) * dk + i] = __expf(b[(n - 1) * dk + i]);
    __syncthreads();
    const int G = GLA_THREADS / dv;
    if (tid >= G * dv) return;
    const int j = tid % dv, g = tid / dv;
    float v[GC];
#pragma unroll
    for (int t = 0; t < GC; t++) v[t] = t < n ? proj[(size_t)(r0 + t) * ld + (size_t)2 * H * dk + (size_t)h * dv + j] : 0.f;
    float *Uc = U + ((size_t)c * H + h) * dk * dv;
    for (int i = g; i < dk; i += G) {
        const float4 *kr = (const float4 *)(kd + i * GC);
        float acc = 0.f;
#pragma unroll
        for (int t4 = 0; t4 < GC / 4; t4++) {
            const float4 k4 = kr[t4];
            acc = fmaf(k4.x, v[4 * t4], acc); acc = fmaf(k4.y, v[4 * t4 + 1], acc);
            acc = fmaf(k4.z, v[4 * t4 + 2], acc); acc = fmaf(k4.w, v[4 * t4 + 3], acc);
        }
        Uc[(size_t)i * dv + j] = acc;
    }
}

// 2. per (sequence, head, slice of the state): S <- D_c S + U_c over the sequence's chunks; U_c receives the state before c.
// Eight chunks' loads are in flight before the eight dependent updates run.
__global__ void __launch_bounds__(GLA_THREADS)
gla_chunk_scan_kernel(float *__restrict__ U, const float *__restrict__ D, const int *__restrict__ seq_chunk0, const int *__restrict__ slots,
                      float *__restrict__ state, int H, int dk, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * GLA_THREADS + threadIdx.x;
    if (e >= dk * dv) return;
    const int i = e / dv;
    const int c0 = seq_chunk0[seq], c1 = seq_chunk0[seq + 1];
    const size_t hs = (size_t)dk * dv;
    float *Sg = state + ((size_t)slots[seq] * H + h) * hs;
    float s = Sg[e];
    for (int c = c0; c < c1; c += 8) {
        float u[8], d[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const bool in = c + k < c1;
            u[k] = in ? U[((size_t)(c + k) * H + h) * hs + e] : 0.f;
            d[k] = in ? D[((size_t)(c + k) * H + h) * dk + i] : 1.f;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (c + k < c1) U[((size_t)(c + k) * H + h) * hs + e] = s;
            s = fmaf(s, d[k], u[k]);
        }
    }
    Sg[e] = s;
}

// 3. outputs of a chunk.  One block per (chunk, head); P (= U after the scan) is the state in front of the chunk.  Thread
// (g, j) owns column j of the chunk's GC outputs (in registers) and, of the sums over key channels and over earlier tokens,
// the terms g, g + G, ...: the state is read ONCE, coalesced, straight from global memory; the groups' partial sums are
// added in group order.
template <typename TO>
__global__ void __launch_bounds__(GLA_THREADS, 3)
gla_chunk_out_kernel(const float *__restrict__ proj, int ld, const float *__restrict__ z, int ldz, const float *__restrict__ z_bias,
                     const float *__restrict__ norm_w, TO *__restrict__ out, int ldo, const int *__restrict__ chunk_row,
                     const int *__restrict__ chunk_len, const float *__restrict__ P, const float *__restrict__ Bg, int H, int dk, int dv,
                     float inv_tau, float q_scale, float eps) {
    extern __shared__ __align__(16) float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int r0 = chunk_row[c], n = chunk_len[c];
    // b, qs, ks: [GC][dk]; qd: [dk][GC] = q_t * exp(b_t), zero beyond n; AT: [GC (u)][GC (t)] = A[t][u], zero where u > t
    float *b = sm, *qs = b + GC * dk, *ks = qs + GC * dk, *qd = ks + GC * dk, *AT = qd + GC * dk, *part = AT + GC * GC, *os = part + GC * GLA_THREADS, *inv = os + GC * dv;
    (void)z; (void)ldz; (void)z_bias; (void)inv_tau;
    for (int e = tid; e < n * dk; e += GLA_THREADS) b[e] = Bg[((size_t)c * H + h) * GC * dk + e];
    const int warp = tid >> 5, lane = tid & 31;
    for (int t = warp; t < n; t += GLA_THREADS / 32) {
        const float *row = proj + (size_t)(r0 + t) * ld;
        for (int i = lane; i < dk; i += 32) {
            qs[t * dk + i] = row[(size_t)h * dk + i] * q_scale;
            ks[t * dk + i] = row[(size_t)(H + h) * dk + i];
        }
    }
    __syncthreads();
    // scores inside the chunk: A[t][u] = sum_i q_t[i] k_u[i] exp(b_t[i] - b_u[i]) for u <= t; a warp per pair
    for (int pair = warp; pair < GC * GC; pair += GLA_THREADS / 32) {
        const int u = pair / GC, t = pair - u * GC;
        if (u > t || t >= n) {                                 // the same for the whole warp
            if (lane == 0) AT[pair] = 0.f;
            continue;
        }
        float acc = 0.f;
        {
            for (int i = lane; i < dk; i += 32) acc = fmaf(qs[t * dk + i] * ks[u * dk + i], __expf(b[t * dk + i] - b[u * dk + i]), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) AT[pair] = acc;
    }
    for (int t = warp; t < GC; t += GLA_THREADS / 32)
        for (int i = lane; i < dk; i += 32) qd[i * GC + t] = t < n ? qs[t * dk + i] * __expf(b[t * dk + i]) : 0.f;
    __syncthreads();
    const int G = GLA_THREADS / dv;
    const bool active = tid < G * dv;
    const int j = tid % dv, g = tid / dv;
    float acc[GC];
#pragma unroll
    for (int t = 0; t < GC; t++) acc[t] = 0.f;
    if (active) {
        const float *Pc = P + ((size_t)c * H + h) * dk * dv;
        // eight rows of the state are requested before the first is used
        for (int i0 = g; i0 < dk; i0 += 8 * G) {
            float p8[8];
#pragma unroll
            for (int k = 0; k < 8; k++) p8[k] = i0 + k * G < dk ? Pc[(size_t)(i0 + k * G) * dv + j] : 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = i0 + k * G;
                if (i >= dk) break;
                const float p = p8[k];
                const float4 *q4 = (const float4 *)(qd + i * GC);
#pragma unroll
                for (int t4 = 0; t4 < GC / 4; t4++) {
                    const float4 w = q4[t4];
                    acc[4 * t4] = fmaf(p, w.x, acc[4 * t4]); acc[4 * t4 + 1] = fmaf(p, w.y, acc[4 * t4 + 1]);
                    acc[4 * t4 + 2] = fmaf(p, w.z, acc[4 * t4 + 2]); acc[4 * t4 + 3] = fmaf(p, w.w, acc[4 * t4 + 3]);
                }
            }
        }
        float vu[GC];                                           // this group's values of column j, requested together
#pragma unroll
        for (int k = 0; k < GC; k++) vu[k] = (g + k * G < n) ? proj[(size_t)(r0 + g + k * G) * ld + (size_t)2 * H * dk + (size_t)h * dv + j] : 0.f;
#pragma unroll
        for (int k = 0; k < GC; k++) {
            const int u = g + k * G;
            if (u >= n) break;
            const float vv = vu[k];
            const float4 *a4 = (const float4 *)(AT + u * GC);
#pragma unroll
            for (int t4 = 0; t4 < GC / 4; t4++) {
                const float4 w = a4[t4];
                acc[4 * t4] = fmaf(vv, w.x, acc[4 * t4]); acc[4 * t4 + 1] = fmaf(vv, w.y, acc[4 * t4 + 1]);
                acc[4 * t4 + 2] = fmaf(vv, w.z, acc[4 * t4 + 2]); acc[4 * t4 + 3] = fmaf(vv, w.w, acc[4 * t4 + 3]);
            }
        }
#pragma unroll
        for (int t = 0; t < GC; t++) part[t * GLA_THREADS + tid] = acc[t];      // [t][g][j]
    }
    __syncthreads();
    // column j's outputs, groups added in order; then the unit norm over the head's values, a warp per token
    // a warp per token: the column sums in group order, the unit norm over the head's values, the gate
    (void)os; (void)inv;
    for (int t = warp; t < n; t += GLA_THREADS / 32) {
        const float *grow = proj + (size_t)(r0 + t) * ld + (size_t)2 * H * dk + (size_t)(H + h) * dv;
        float ss = 0.f;
        for (int jj = lane; jj < dv; jj += 32) {
            float o = 0.f;
            for (int gg = 0; gg < G; gg++) o += part[t * GLA_THREADS + gg * dv + jj];
            part[t * GLA_THREADS + jj] = o;                     // group 0's place: read and written by this lane alone
            ss = fmaf(o, o, ss);
        }
        ss = warp_sum(ss);
        const float inv_t = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int jj = lane; jj < dv; jj += 32)
            out[(size_t)(r0 + t) * ldo + (size_t)h * dv + jj] = from_f32<TO>(part[t * GLA_THREADS + jj] * inv_t * norm_w[jj] * gla_silu(grow[jj]));
    }
}

static FgPerDevice g_gla_seq_setup[2], g_gla_state_setup, g_gla_out_setup[2];

static size_t gla_seq_smem(int dk, int dv) { return ((size_t)dk * dv + 3 * dk + dv + (size_t)(GLA_THREADS / dv) * dv) * sizeof(float); }
static size_t gla_state_smem(int dk, int dv) { (void)dv; return (size_t)2 * GC * dk * sizeof(float); }
static size_t gla_out_smem(int dk, int dv) {
    return ((size_t)4 * GC * dk + (size_t)GC * dv + GC * GC + (size_t)GC * GLA_THREADS + GC) * sizeof(float);
}

extern "C" int fg_gla_chunk_tokens(void) { return GC; }

extern "C" int fg_gla(const float *proj, int ld, const float *z, int ldz, const float *z_bias, const float *norm_w, void *out, int out_dtype,
                      int ldo, const int *cu_rows, const int *slots, float *state, int n_seq, int H, int dk, int dv, float tau, float q_scale,
                      float eps, cudaStream_t stream) {
    if (n_seq <= 0) return 0;
    if (dk <= 0 || dv <= 0 || dv > GLA_THREADS || H <= 0 || H > 65535 || !(tau > 0.f)) return FG_ERR_BAD_SIZE;
    const size_t smem = gla_seq_smem(dk, dv);
    if (smem > 200 * 1024) return FG_ERR_BAD_SIZE;
    if (out_dtype != FG_F32 && out_dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
    const bool wide = out_dtype == FG_F32;
    if (fg_needs_setup(g_gla_seq_setup[wide ? 0 : 1])) {
        cudaError_t e = wide ? cudaFuncSetAttribute(gla_seq_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                             : cudaFuncSetAttribute(gla_seq_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    if (wide)
        return fg_launch(gla_seq_kernel<float>, dim3(n_seq, H), dim3(GLA_THREADS), smem, stream, proj, ld, z, ldz, z_bias, norm_w, (float *)out,
                         ldo, cu_rows, slots, state, H, dk, dv, 1.0f / tau, q_scale, eps);
    return fg_launch(gla_seq_kernel<bf16>, dim3(n_seq, H), dim3(GLA_THREADS), smem, stream, proj, ld, z, ldz, z_bias, norm_w, (bf16 *)out, ldo,
                     cu_rows, slots, state, H, dk, dv, 1.0f / tau, q_scale, eps);
}

// 1 if the chunked form takes these sizes
extern "C" int fg_gla_chunked_ok(int dk, int dv) {
    if (dk <= 0 || dv <= 0 || dv > GLA_THREADS) return 0;
    return gla_state_smem(dk, dv) <= 200 * 1024 && gla_out_smem(dk, dv) <= 200 * 1024;
}

// n_chunks = sum over sequences of ceil(rows / fg_gla_chunk_tokens()).  plan: scratch of 2 * n_chunks + n_seq + 1 ints;
// U: scratch [n_chunks, H, dk, dv] float32; D: scratch [n_chunks, H, dk (1 + chunk tokens)] float32 (the chunks' decays, then the
// cumulative log decays of their tokens).
extern "C" int fg_gla_chunked(const float *proj, int ld, const float *z, int ldz, const float *z_bias, const float *norm_w, void *out,
                              int out_dtype, int ldo, const int *cu_rows, const int *slots, float *state, int *plan, float *U, float *D,
                              int n_seq, int n_chunks, int H, int dk, int dv, float tau, float q_scale, float eps, cudaStream_t stream) {
    if (n_seq <= 0 || n_chunks <= 0) return 0;
    if (!fg_gla_chunked_ok(dk, dv) || H <= 0 || H > 65535 || !(tau > 0.f)) return FG_ERR_BAD_SIZE;
    if (out_dtype != FG_F32 && out_dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
    const bool wide = out_dtype == FG_F32;
    if (fg_needs_setup(g_gla_state_setup)) {
        cudaError_t e = cudaFuncSetAttribute(gla_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    if (fg_needs_setup(g_gla_out_setup[wide ? 0 : 1])) {
        cudaError_t e = wide ? cudaFuncSetAttribute(gla_chunk_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                             : cudaFuncSetAttribute(gla_chunk_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    int *chunk_row = plan, *chunk_len = plan + n_chunks, *seq_chunk0 = plan + 2 * n_chunks;
    const float inv_tau = 1.0f / tau;
    int code = fg_launch(gla_chunk_plan_kernel, dim3(1), dim3(n_seq >= 256 ? 256 : 32), 0, stream, cu_rows, n_seq, chunk_row, chunk_len, seq_chunk0);
    if (code) return code;
    float *Bg = D + (size_t)n_chunks * H * dk;
    code = fg_launch(gla_chunk_state_kernel, dim3(n_chunks, H), dim3(GLA_THREADS), gla_state_smem(dk, dv), stream, proj, ld, z, ldz, z_bias,
                     (const int *)chunk_row, (const int *)chunk_len, U, D, Bg, H, dk, dv, inv_tau);
    if (code) return code;
    code = fg_launch(gla_chunk_scan_kernel, dim3(n_seq, H, (dk * dv + GLA_THREADS - 1) / GLA_THREADS), dim3(GLA_THREADS), 0, stream, U,
                     (const float *)D, (const int *)seq_chunk0, slots, state, H, dk, dv);
    if (code) return code;
    if (wide)
        return fg_launch(gla_chunk_out_kernel<float>, dim3(n_chunks, H), dim3(GLA_THREADS), gla_out_smem(dk, dv), stream, proj, ld, z, ldz, z_bias,
                         norm_w, (float *)out, ldo, (const int *)chunk_row, (const int *)chunk_len, (const float *)U, (const float *)Bg, H, dk, dv, inv_tau,
                         q_scale, eps);
    return fg_launch(gla_chunk_out_kernel<bf16>, dim3(n_chunks, H), dim3(GLA_THREADS), gla_out_smem(dk, dv), stream, proj, ld, z, ldz, z_bias,
                     norm_w, (bf16 *)out, ldo, (const int *)chunk_row, (const int *)chunk_len, (const float *)U, (const float *)Bg, H, dk, dv, inv_tau,
                     q_scale, eps);
}
