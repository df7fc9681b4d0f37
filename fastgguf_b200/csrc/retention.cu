// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
// Per head, with q_t, k_t (rotated; k times k_scale afterwards) of size dk and v_t of size dv:
//     S_t = decay * S_(t-1) + k_t v_t^T          (S: [dk, dv], zero at the start of a sequence)
//     o_t = S_t^T q_t
//     y_t = o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)
// The state S, the rotation, the decay powers, the scores and the unit norm are 32-bit in every engine dtype; S lives
// in the engine's per-sequence state rows [slot, H, dk, dv] and is carried from step to step.
//
// A row of `proj` holds the four projections of a token: q [H, dk] | k [H, dk] | v [H, dv] | g [H, dv], float32.
// Rotation tables cos/sin are [positions, dk / 2] for pairs (j, j + dk / 2); dimensions that are not rotated have
// cos 1, sin 0 (the rows of the q and k projections are permuted into that form when the weights are loaded).
//
// Two forms:
//   * retention_seq_kernel: one block per (sequence, head) walks its tokens one after another with S in shared memory.
//     A decode step (one token a sequence) and short portions run this way.
//   * the chunked form for long portions, three kernels over chunks of RC tokens, all chunks of all sequences at once:
//       1. U_c = sum_j decay^(n-1-j) k_j v_j^T              what chunk c (n tokens) adds to the state
//       2. S_c = decay^n S_(c-1) + U_c, chunk after chunk    (U_c is overwritten by the state BEFORE chunk c)
//       3. o_i = decay^(i+1) S_(c-1)^T q_i + sum_(j<=i) decay^(i-j) (q_i . k_j) v_j, then unit norm and gate
//     The sums are the recurrence's own terms in another order; nothing is approximated.
#include "common.cuh"

#define RET_THREADS 256
#define RC 32                       // tokens a chunk

template <typename TO> __device__ __forceinline__ void store4(TO *dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float *dst, float a, float b, float c, float d) {
    *(float4 *)dst = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16 *dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *(uint2 *)dst = make_uint2(*(uint32_t *)&lo, *(uint32_t *)&hi);
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// rotate pair (j, j + half) of head vector `src` at position pos into dst (shared memory), times `mul`
__device__ __forceinline__ void rotate_into(const float *__restrict__ src, float *dst, int dk, const float *cs, const float *sn,
                                            float mul, int tid, int nthreads) {
    const int half = dk >> 1;
    for (int j = tid; j < half; j += nthreads) {
        float a = src[j], b = src[j + half], c = cs[j], s = sn[j];
        dst[j] = (a * c - b * s) * mul;
        dst[j + half] = (b * c + a * s) * mul;
    }
}

// The same for the n tokens of a chunk at once, all threads busy and many loads in flight: dst[t][..] (row stride
// `stride`) = rotated head vector of token r0 + t, times mul (and, DECAY, times decay^(n - 1 - t)).
template <bool DECAY>
__device__ __forceinline__ void rotate_chunk_into(const float *__restrict__ proj, int ld, int r0, int n, size_t head_off, float *dst,
                                                  int stride, int dk, const int *__restrict__ positions,
                                                  const float *__restrict__ cos_t, const float *__restrict__ sin_t, float mul, float l2,
                                                  int tid) {
    const int half = dk >> 1;
#pragma unroll 4
    for (int e = tid; e < n * half; e += RET_THREADS) {
        const int t = e / half, j = e - t * half;
        const float *src = proj + (size_t)(r0 + t) * ld + head_off;
        const int pos = positions[r0 + t];
        const float a = src[j], b = src[j + half], c = cos_t[(size_t)pos * half + j], sn = sin_t[(size_t)pos * half + j];
        const float m = DECAY ? mul * exp2f(l2 * (float)(n - 1 - t)) : mul;
        dst[t * stride + j] = (a * c - b * sn) * m;
        dst[t * stride + j + half] = (b * c + a * sn) * m;
    }
}
__device__ __forceinline__ void copy_chunk_into(const float *__restrict__ proj, int ld, int r0, int n, size_t off, float *dst, int dv, int tid) {
#pragma unroll 4
    for (int e = tid; e < n * dv; e += RET_THREADS) {
        const int t = e / dv, j = e - t * dv;
        dst[e] = proj[(size_t)(r0 + t) * ld + off + j];
    }
}

template <typename TO>
__global__ void __launch_bounds__(RET_THREADS)
retention_seq_kernel(const float *__restrict__ proj, int ld, TO *__restrict__ out, int ldo, const int *__restrict__ positions,
                     const int *__restrict__ cu_rows, const int *__restrict__ slots, const float *__restrict__ cos_t,
                     const float *__restrict__ sin_t, const float *__restrict__ decay, float *__restrict__ state, int H, int dk,
                     int dv, float k_scale, float eps) {
    extern __shared__ float sm[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = cu_rows[seq], row1 = cu_rows[seq + 1];
    if (row1 <= row0) return;
    const int G = RET_THREADS / dv, n_active = G * dv;      // threads (g, j): column j of S, rows g, g + G, ...
    float *S = sm, *qs = S + dk * dv, *ks = qs + dk, *vs = ks + dk, *part = vs + dv;
    float *Sg = state + ((size_t)slots[seq] * H + h) * dk * dv;
    for (int e = tid; e < dk * dv; e += RET_THREADS) S[e] = Sg[e];
    const float dec = decay[h];
    const int half = dk >> 1;
    for (int r = row0; r < row1; r++) {
        const float *row = proj + (size_t)r * ld;
        const int pos = positions[r];
        const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
        rotate_into(row + (size_t)h * dk, qs, dk, cs, sn, 1.0f, tid, RET_THREADS);
        rotate_into(row + (size_t)(H + h) * dk, ks, dk, cs, sn, k_scale, tid, RET_THREADS);
        for (int j = tid; j < dv; j += RET_THREADS) vs[j] = row[(size_t)2 * H * dk + (size_t)h * dv + j];
        __syncthreads();
        if (tid < n_active) {
            const int j = tid % dv, g = tid / dv;
            const float vj = vs[j];
            float acc = 0.f;
            for (int i = g; i < dk; i += G) {
                float s = fmaf(S[i * dv + j], dec, ks[i] * vj);
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
            out[(size_t)r * ldo + (size_t)h * dv + tid] = from_f32<TO>(o * (1.0f / sqrtf(ss / (float)dv + eps)) * silu_f(gate));
        }
    }
    __syncthreads();
    for (int e = tid; e < dk * dv; e += RET_THREADS) Sg[e] = S[e];
}

// ------------------------------------------------------------------ chunked form
// Chunk c of the step covers tokens [chunk_row[c], chunk_row[c] + chunk_len[c]); the chunks of a sequence are consecutive
// and in order, sequence s owning chunks [seq_chunk0[s], seq_chunk0[s + 1]).  The plan is made on the device from the
// step's row offsets; the host only knows how many chunks there are.
__global__ void retention_chunk_plan_kernel(const int *__restrict__ cu_rows, int n_seq, int *__restrict__ chunk_row,
                                            int *__restrict__ chunk_len, int *__restrict__ seq_chunk0) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int s = 0; s < n_seq; s++) { seq_chunk0[s] = at; at += (cu_rows[s + 1] - cu_rows[s] + RC - 1) / RC; }
        seq_chunk0[n_seq] = at;
    }
    __syncthreads();
    for (int s = threadIdx.x; s < n_seq; s += blockDim.x) {
        const int r0 = cu_rows[s], r1 = cu_rows[s + 1];
        int c = seq_chunk0[s];
        for (int r = r0; r < r1; r += RC, c++) { chunk_row[c] = r; chunk_len[c] = min(RC, r1 - r); }
    }
}

// 1. U[c, h] = sum_j decay^(n-1-j) k_j v_j^T.  One block per (chunk, head); thread (g, j) owns column j, rows g, g + G, ...
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_state_kernel(const float *__restrict__ proj, int ld, const int *__restrict__ positions,
                             const int *__restrict__ chunk_row, const int *__restrict__ chunk_len,
                             const float *__restrict__ cos_t, const float *__restrict__ sin_t, const float *__restrict__ decay,
                             float *__restrict__ U, int H, int dk, int dv, float k_scale) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int r0 = chunk_row[c], n = chunk_len[c];
    float *K = sm, *V = K + RC * dk;            // K[t][dk] carries decay^(n-1-t); V[t][dv]
    const int half = dk >> 1;
    const float l2 = log2f(decay[h]);
    for (int t = 0; t < n; t++) {
        const float *row = proj + (size_t)(r0 + t) * ld;
        const int pos = positions[r0 + t];
        rotate_into(row + (size_t)(H + h) * dk, K + t * dk, dk, cos_t + (size_t)pos * half, sin_t + (size_t)pos * half,
                    k_scale * exp2f(l2 * (float)(n - 1 - t)), tid, RET_THREADS);
        for (int j = tid; j < dv; j += RET_THREADS) V[t * dv + j] = row[(size_t)2 * H * dk + (size_t)h * dv + j];
    }
    __syncthreads();
    const int G = RET_THREADS / dv;
    if (tid >= G * dv) return;
    const int j = tid % dv, g = tid / dv;
    float *Ug = U + ((size_t)c * H + h) * dk * dv;
    for (int i = g; i < dk; i += G) {
        float acc = 0.f;
        for (int t = 0; t < n; t++) acc = fmaf(K[t * dk + i], V[t * dv + j], acc);
        Ug[i * dv + j] = acc;
    }
}

// 2. The scan over a sequence's chunks, element by element: U[c] <- state before chunk c; the state after the last chunk
//    goes back to the sequence's state row.  grid (sequences, heads, slices of dk * dv).
template <typename V>          // V = float4 where a head's state is a multiple of four floats (16-byte accesses), else float
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_scan_kernel(const int *__restrict__ seq_chunk0, const int *__restrict__ chunk_len, const int *__restrict__ slots,
                            const float *__restrict__ decay, float *__restrict__ U, float *__restrict__ state, int H, int dk, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int W = sizeof(V) / sizeof(float);
    const int seq = blockIdx.x, h = blockIdx.y;
    const int e = (blockIdx.z * RET_THREADS + threadIdx.x) * W;
    if (e >= dk * dv) return;
    const int c0 = seq_chunk0[seq], c1 = seq_chunk0[seq + 1];
    if (c1 <= c0) return;
    V *Sg = (V *)(state + ((size_t)slots[seq] * H + h) * dk * dv + e);
    const float l2 = log2f(decay[h]);
    V sv = *Sg;
    float *s = (float *)&sv;
    const size_t step = (size_t)H * dk * dv;
    float *u = U + ((size_t)c0 * H + h) * dk * dv + e;
    for (int c = c0; c < c1; c += 8) {
        // eight chunks' contributions are fetched before the first is used: the chain of sums does not wait for memory
        V add[8];
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (c + i < c1) add[i] = *(const V *)(u + (size_t)i * step);
            f[i] = c + i < c1 ? exp2f(l2 * (float)chunk_len[c + i]) : 1.f;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (c + i >= c1) break;
            *(V *)(u + (size_t)i * step) = sv;
            const float *a = (const float *)&add[i];
#pragma unroll
            for (int w = 0; w < W; w++) s[w] = fmaf(s[w], f[i], a[w]);
        }
        u += 8 * step;
    }
    *Sg = sv;
}

// 3. Outputs of a chunk.  One block per (chunk, head): A[i][j] = decay^(i-j) (q_i . k_j) for j <= i, then
//    o_i = decay^(i+1) S^T q_i + sum_j A[i][j] v_j, unit norm over dv, times silu(g).
template <typename TO>
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_out_kernel(const float *__restrict__ proj, int ld, TO *__restrict__ out, int ldo, const int *__restrict__ positions,
                           const int *__restrict__ chunk_row, const int *__restrict__ chunk_len, const float *__restrict__ cos_t,
                           const float *__restrict__ sin_t, const float *__restrict__ decay, const float *__restrict__ U, int H,
                           int dk, int dv, float k_scale, float eps) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int r0 = chunk_row[c], n = chunk_len[c];
    const int dkp = dk + 1;                      // padded rows: threads of a warp read different rows of Q / K
    float *Q = sm, *K = Q + RC * dkp, *V = K + RC * dkp, *A = V + RC * dv, *O = A + RC * RC, *inv = O + RC * dv;
    const int half = dk >> 1;
    const float l2 = log2f(decay[h]);
    for (int t = 0; t < n; t++) {
        const float *row = proj + (size_t)(r0 + t) * ld;
        const int pos = positions[r0 + t];
        const float *cs = cos_t + (size_t)pos * half, *sn = sin_t + (size_t)pos * half;
        rotate_into(row + (size_t)h * dk, Q + t * dkp, dk, cs, sn, 1.0f, tid, RET_THREADS);
        rotate_into(row + (size_t)(H + h) * dk, K + t * dkp, dk, cs, sn, k_scale, tid, RET_THREADS);
        for (int j = tid; j < dv; j += RET_THREADS) V[t * dv + j] = row[(size_t)2 * H * dk + (size_t)h * dv + j];
    }
    __syncthreads();
    for (int e = tid; e < n * RC; e += RET_THREADS) {
        const int i = e / RC, j = e % RC;
        float a = 0.f;
        if (j <= i) {
            for (int d = 0; d < dk; d++) a = fmaf(Q[i * dkp + d], K[j * dkp + d], a);
            a *= exp2f(l2 * (float)(i - j));
        }
        A[e] = a;
    }
    __syncthreads();
    // thread (g, j): column j of the output, tokens g, g + G, ...
    const int G = RET_THREADS / dv;
    const float *S = U + ((size_t)c * H + h) * dk * dv;
    if (tid < G * dv) {
        const int j = tid % dv, g = tid / dv;
        for (int i0 = g; i0 < n; i0 += 4 * G) {
            // four tokens at a time share each element of S
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            const int ii[4] = {i0, i0 + G, i0 + 2 * G, i0 + 3 * G};
            for (int d = 0; d < dk; d++) {
                const float s = S[d * dv + j];
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (ii[u] < n) acc[u] = fmaf(Q[ii[u] * dkp + d], s, acc[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (ii[u] >= n) continue;
                float o = acc[u] * exp2f(l2 * (float)(ii[u] + 1));
                for (int t = 0; t <= ii[u]; t++) o = fmaf(A[ii[u] * RC + t], V[t * dv + j], o);
                O[ii[u] * dv + j] = o;
            }
        }
    }
    __syncthreads();
    // unit norm of each token's head vector: a warp per token
    const int warp = tid >> 5, lane = tid & 31;
    for (int i = warp; i < n; i += RET_THREADS / 32) {
        float ss = 0.f;
        for (int j = lane; j < dv; j += 32) ss = fmaf(O[i * dv + j], O[i * dv + j], ss);
        ss = warp_sum(ss);
        if (lane == 0) inv[i] = 1.0f / sqrtf(ss / (float)dv + eps);
    }
    __syncthreads();
    for (int e = tid; e < n * dv; e += RET_THREADS) {
        const int i = e / dv, j = e % dv;
        const float gate = proj[(size_t)(r0 + i) * ld + (size_t)2 * H * dk + (size_t)(H + h) * dv + j];
        out[(size_t)(r0 + i) * ldo + (size_t)h * dv + j] = from_f32<TO>(O[e] * inv[i] * silu_f(gate));
    }
}

// ------------------------------------------------------------------ the chunked form with register tiles
// The same three steps for head sizes 64 and 128 (keys and values each), where the tiles divide evenly: every thread
// owns a small tile of the result and reads its operands sixteen bytes at a time, so that the FMA units, not the
// load units, set the pace.  Sums run over the same terms in the same order as in the plain kernels above.

// 1. U = K'^T V.  Thread (ti, tj): rows ti * TI .. + TI of U, columns tj * 4 .. + 4.
template <int DK, int DV>
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_state_fast(const float *__restrict__ proj, int ld, const int *__restrict__ positions,
                           const int *__restrict__ chunk_row, const int *__restrict__ chunk_len,
                           const float *__restrict__ cos_t, const float *__restrict__ sin_t, const float *__restrict__ decay,
                           float *__restrict__ U, int H, float k_scale) {
    constexpr int NJ = DV / 4, NI = RET_THREADS / NJ, TI = DK / NI;
    __shared__ __align__(16) float K[RC * DK];
    __shared__ __align__(16) float V[RC * DV];
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int r0 = chunk_row[c], n = chunk_len[c];
    const float l2 = log2f(decay[h]);
    rotate_chunk_into<true>(proj, ld, r0, n, (size_t)(H + h) * DK, K, DK, DK, positions, cos_t, sin_t, k_scale, l2, tid);
    copy_chunk_into(proj, ld, r0, n, (size_t)2 * H * DK + (size_t)h * DV, V, DV, tid);
    __syncthreads();
    const int tj = tid % NJ, ti = tid / NJ;
    float acc[TI][4];
#pragma unroll
    for (int u = 0; u < TI; u++) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
    for (int t = 0; t < n; t++) {
        const float4 v = *(const float4 *)(V + t * DV + tj * 4);
        float k[TI];
#pragma unroll
        for (int u = 0; u < TI; u += 4) *(float4 *)(k + u) = *(const float4 *)(K + t * DK + ti * TI + u);
#pragma unroll
        for (int u = 0; u < TI; u++) {
            acc[u][0] = fmaf(k[u], v.x, acc[u][0]); acc[u][1] = fmaf(k[u], v.y, acc[u][1]);
            acc[u][2] = fmaf(k[u], v.z, acc[u][2]); acc[u][3] = fmaf(k[u], v.w, acc[u][3]);
        }
    }
    float *Ug = U + ((size_t)c * H + h) * DK * DV;
#pragma unroll
    for (int u = 0; u < TI; u++) *(float4 *)(Ug + (size_t)(ti * TI + u) * DV + tj * 4) = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
}

// 3. Outputs.  Thread (ti, tj): tokens ti, ti + NI, ..., columns tj * 4 .. + 4; a token's row lies in NJ neighbouring lanes.
template <int DK, int DV, typename TO>
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_out_fast(const float *__restrict__ proj, int ld, TO *__restrict__ out, int ldo, const int *__restrict__ positions,
                         const int *__restrict__ chunk_row, const int *__restrict__ chunk_len, const float *__restrict__ cos_t,
                         const float *__restrict__ sin_t, const float *__restrict__ decay, const float *__restrict__ U, int H,
                         float k_scale, float eps) {
    constexpr int NJ = DV / 4, NI = RET_THREADS / NJ, TT = RC / NI, DKP = DK + 4;
    extern __shared__ __align__(16) float sm[];
    float *Q = sm, *K = Q + RC * DKP, *V = K + RC * DKP, *A = V + RC * DV;       // Q, K: [RC][DKP]; V: [RC][DV]; A: [RC][RC]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int r0 = chunk_row[c], n = chunk_len[c];
    const float l2 = log2f(decay[h]);
    rotate_chunk_into<false>(proj, ld, r0, n, (size_t)h * DK, Q, DKP, DK, positions, cos_t, sin_t, 1.0f, 0.f, tid);
    rotate_chunk_into<false>(proj, ld, r0, n, (size_t)(H + h) * DK, K, DKP, DK, positions, cos_t, sin_t, k_scale, 0.f, tid);
    copy_chunk_into(proj, ld, r0, n, (size_t)2 * H * DK + (size_t)h * DV, V, DV, tid);
    for (int e = n * DKP + tid; e < RC * DKP; e += RET_THREADS) Q[e] = K[e] = 0.f;       // rows of a short last chunk
    for (int e = n * DV + tid; e < RC * DV; e += RET_THREADS) V[e] = 0.f;
    __syncthreads();
    // scores: four (i, j) pairs a thread
    for (int e = tid; e < RC * RC; e += RET_THREADS) {
        const int i = e / RC, j = e % RC;
        float a = 0.f;
        if (j <= i && i < n) {
#pragma unroll 8
            for (int d = 0; d < DK; d += 4) {
                const float4 q = *(const float4 *)(Q + i * DKP + d), k = *(const float4 *)(K + j * DKP + d);
                a = fmaf(q.x, k.x, a); a = fmaf(q.y, k.y, a); a = fmaf(q.z, k.z, a); a = fmaf(q.w, k.w, a);
            }
            a *= exp2f(l2 * (float)(i - j));
        }
        A[e] = a;
    }
    __syncthreads();
    const int tj = tid % NJ, ti = tid / NJ;
    const float *S = U + ((size_t)c * H + h) * DK * DV + tj * 4;
    float acc[TT][4];
#pragma unroll
    for (int u = 0; u < TT; u++) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
    // what the state before the chunk gives: Q S, four rows of S at a time
#pragma unroll 4
    for (int d = 0; d < DK; d += 4) {
        const float4 s0 = *(const float4 *)(S + (size_t)d * DV), s1 = *(const float4 *)(S + (size_t)(d + 1) * DV);
        const float4 s2 = *(const float4 *)(S + (size_t)(d + 2) * DV), s3 = *(const float4 *)(S + (size_t)(d + 3) * DV);
#pragma unroll
        for (int u = 0; u < TT; u++) {
            const float4 q = *(const float4 *)(Q + (ti + u * NI) * DKP + d);
            acc[u][0] = fmaf(q.x, s0.x, acc[u][0]); acc[u][1] = fmaf(q.x, s0.y, acc[u][1]); acc[u][2] = fmaf(q.x, s0.z, acc[u][2]); acc[u][3] = fmaf(q.x, s0.w, acc[u][3]);
            acc[u][0] = fmaf(q.y, s1.x, acc[u][0]); acc[u][1] = fmaf(q.y, s1.y, acc[u][1]); acc[u][2] = fmaf(q.y, s1.z, acc[u][2]); acc[u][3] = fmaf(q.y, s1.w, acc[u][3]);
            acc[u][0] = fmaf(q.z, s2.x, acc[u][0]); acc[u][1] = fmaf(q.z, s2.y, acc[u][1]); acc[u][2] = fmaf(q.z, s2.z, acc[u][2]); acc[u][3] = fmaf(q.z, s2.w, acc[u][3]);
            acc[u][0] = fmaf(q.w, s3.x, acc[u][0]); acc[u][1] = fmaf(q.w, s3.y, acc[u][1]); acc[u][2] = fmaf(q.w, s3.z, acc[u][2]); acc[u][3] = fmaf(q.w, s3.w, acc[u][3]);
        }
    }
#pragma unroll
    for (int u = 0; u < TT; u++) {
        const float f = exp2f(l2 * (float)(ti + u * NI + 1));
        acc[u][0] *= f; acc[u][1] *= f; acc[u][2] *= f; acc[u][3] *= f;
    }
    // what the chunk's own tokens give: A V (A is zero beyond a token's own place)
    for (int t = 0; t < n; t++) {
        const float4 v = *(const float4 *)(V + t * DV + tj * 4);
#pragma unroll
        for (int u = 0; u < TT; u++) {
            const float a = A[(ti + u * NI) * RC + t];
            acc[u][0] = fmaf(a, v.x, acc[u][0]); acc[u][1] = fmaf(a, v.y, acc[u][1]); acc[u][2] = fmaf(a, v.z, acc[u][2]); acc[u][3] = fmaf(a, v.w, acc[u][3]);
        }
    }
    // unit norm over the head's values (NJ neighbouring lanes hold a token's row), gate, store
#pragma unroll
    for (int u = 0; u < TT; u++) {
        const int i = ti + u * NI;
        float ss = acc[u][0] * acc[u][0] + acc[u][1] * acc[u][1] + acc[u][2] * acc[u][2] + acc[u][3] * acc[u][3];
#pragma unroll
        for (int o = NJ / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (i >= n) continue;
        const float inv = 1.0f / sqrtf(ss / (float)DV + eps);
        const float4 g = *(const float4 *)(proj + (size_t)(r0 + i) * ld + (size_t)2 * H * DK + (size_t)(H + h) * DV + tj * 4);
        TO *o = out + (size_t)(r0 + i) * ldo + (size_t)h * DV + tj * 4;
        store4<TO>(o, acc[u][0] * inv * silu_f(g.x), acc[u][1] * inv * silu_f(g.y), acc[u][2] * inv * silu_f(g.z), acc[u][3] * inv * silu_f(g.w));
    }
}

// ------------------------------------------------------------------ launchers
static FgPerDevice g_seq_setup[2], g_state_setup, g_out_setup[2];

extern "C" int fg_retention_chunk_tokens(void) { return RC; }

extern "C" int fg_retention(const float *proj, int ld, void *out, int out_dtype, int ldo, const int *positions, const int *cu_rows,
                            const int *slots, const float *cos_t, const float *sin_t, const float *decay, float *state, int n_seq,
                            int H, int dk, int dv, float k_scale, float eps, cudaStream_t stream) {
    if (n_seq <= 0) return 0;
    if (dk <= 0 || dk % 2 || dv <= 0 || dv > RET_THREADS || H <= 0 || H > 65535) return FG_ERR_BAD_SIZE;
    const int G = RET_THREADS / dv;
    size_t smem = ((size_t)dk * dv + 2 * dk + dv + (size_t)G * dv) * sizeof(float);
    if (smem > 200 * 1024) return FG_ERR_BAD_SIZE;
    if (out_dtype != FG_F32 && out_dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
    const bool wide = out_dtype == FG_F32;
    if (fg_needs_setup(g_seq_setup[wide ? 0 : 1])) {
        cudaError_t e = wide ? cudaFuncSetAttribute(retention_seq_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                             : cudaFuncSetAttribute(retention_seq_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    if (wide)
        return fg_launch(retention_seq_kernel<float>, dim3(n_seq, H), dim3(RET_THREADS), smem, stream, proj, ld, (float *)out, ldo,
                         positions, cu_rows, slots, cos_t, sin_t, decay, state, H, dk, dv, k_scale, eps);
    return fg_launch(retention_seq_kernel<bf16>, dim3(n_seq, H), dim3(RET_THREADS), smem, stream, proj, ld, (bf16 *)out, ldo, positions,
                     cu_rows, slots, cos_t, sin_t, decay, state, H, dk, dv, k_scale, eps);
}

// 0 if the chunked form takes these sizes
extern "C" int fg_retention_chunked_ok(int dk, int dv) {
    if (dk <= 0 || dk % 2 || dv <= 0 || dv > RET_THREADS) return 0;
    size_t s1 = (size_t)RC * (dk + dv) * 4;
    size_t s3 = ((size_t)2 * RC * (dk + 1) + 2 * (size_t)RC * dv + RC * RC + RC) * 4;
    return s1 <= 200 * 1024 && s3 <= 200 * 1024;
}

// n_chunks = sum over sequences of ceil(rows / fg_retention_chunk_tokens()).  plan: scratch of 2 * n_chunks + n_seq + 1
// ints; U: scratch [n_chunks, H, dk, dv] float32.
extern "C" int fg_retention_chunked(const float *proj, int ld, void *out, int out_dtype, int ldo, const int *positions,
                                    const int *cu_rows, const int *slots, const float *cos_t, const float *sin_t,
                                    const float *decay, float *state, int *plan, float *U, int n_seq, int n_chunks, int H, int dk,
                                    int dv, float k_scale, float eps, cudaStream_t stream) {
    if (n_seq <= 0 || n_chunks <= 0) return 0;
    if (!fg_retention_chunked_ok(dk, dv) || H <= 0 || H > 65535) return FG_ERR_BAD_SIZE;
    if (out_dtype != FG_F32 && out_dtype != FG_BF16) return FG_ERR_BAD_DTYPE;
    const bool wide = out_dtype == FG_F32;
    size_t s1 = (size_t)RC * (dk + dv) * 4;
    size_t s3 = ((size_t)2 * RC * (dk + 1) + 2 * (size_t)RC * dv + RC * RC + RC) * 4;
    if (fg_needs_setup(g_state_setup)) {
        cudaError_t e = cudaFuncSetAttribute(retention_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    if (fg_needs_setup(g_out_setup[wide ? 0 : 1])) {
        cudaError_t e = wide ? cudaFuncSetAttribute(retention_chunk_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                             : cudaFuncSetAttribute(retention_chunk_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    int *chunk_row = plan, *chunk_len = plan + n_chunks, *seq_chunk0 = plan + 2 * n_chunks;
    // head sizes 64 / 128 with 16-byte aligned rows: the kernels with register tiles
    const bool fast = (dk == 64 || dk == 128) && (dv == 64 || dv == 128) && ld % 4 == 0 && (((uintptr_t)proj | (uintptr_t)U) & 15) == 0 &&
                      ldo % 4 == 0 && ((uintptr_t)out & 15) == 0;
    int code = fg_launch(retention_chunk_plan_kernel, dim3(1), dim3(n_seq >= 256 ? 256 : 32), 0, stream, cu_rows, n_seq, chunk_row, chunk_len,
                         seq_chunk0);
    if (code) return code;
#define RET_STATE_FAST(DK, DV) fg_launch(retention_chunk_state_fast<DK, DV>, dim3(n_chunks, H), dim3(RET_THREADS), 0, stream, proj, ld, positions, \
        (const int *)chunk_row, (const int *)chunk_len, cos_t, sin_t, decay, U, H, k_scale)
    if (fast) code = dk == 64 ? (dv == 64 ? RET_STATE_FAST(64, 64) : RET_STATE_FAST(64, 128)) : (dv == 64 ? RET_STATE_FAST(128, 64) : RET_STATE_FAST(128, 128));
    else code = fg_launch(retention_chunk_state_kernel, dim3(n_chunks, H), dim3(RET_THREADS), s1, stream, proj, ld, positions, (const int *)chunk_row,
                          (const int *)chunk_len, cos_t, sin_t, decay, U, H, dk, dv, k_scale);
#undef RET_STATE_FAST
    if (code) return code;
    if ((dk * dv) % 4 == 0 && (((uintptr_t)U | (uintptr_t)state) & 15) == 0)
        code = fg_launch(retention_chunk_scan_kernel<float4>, dim3(n_seq, H, (dk * dv / 4 + RET_THREADS - 1) / RET_THREADS), dim3(RET_THREADS), 0,
                         stream, (const int *)seq_chunk0, (const int *)chunk_len, slots, decay, U, state, H, dk, dv);
    else
        code = fg_launch(retention_chunk_scan_kernel<float>, dim3(n_seq, H, (dk * dv + RET_THREADS - 1) / RET_THREADS), dim3(RET_THREADS), 0, stream,
                         (const int *)seq_chunk0, (const int *)chunk_len, slots, decay, U, state, H, dk, dv);
    if (code) return code;
    if (fast) {
        const size_t sf = ((size_t)2 * RC * (dk + 4) + (size_t)RC * dv + RC * RC) * sizeof(float);
#define RET_OUT_FAST(DK, DV, TO) do { \
        static FgPerDevice setup; \
        if (fg_needs_setup(setup)) { \
            cudaError_t e = cudaFuncSetAttribute(retention_chunk_out_fast<DK, DV, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
            if (e != cudaSuccess) return (int)e; \
        } \
        return fg_launch(retention_chunk_out_fast<DK, DV, TO>, dim3(n_chunks, H), dim3(RET_THREADS), sf, stream, proj, ld, (TO *)out, ldo, positions, \
                         (const int *)chunk_row, (const int *)chunk_len, cos_t, sin_t, decay, (const float *)U, H, k_scale, eps); } while (0)
#define RET_OUT_FAST_T(TO) do { \
        if (dk == 64 && dv == 64) RET_OUT_FAST(64, 64, TO); \
        if (dk == 64 && dv == 128) RET_OUT_FAST(64, 128, TO); \
        if (dk == 128 && dv == 64) RET_OUT_FAST(128, 64, TO); \
        RET_OUT_FAST(128, 128, TO); } while (0)
        if (wide) RET_OUT_FAST_T(float);
        RET_OUT_FAST_T(bf16);
#undef RET_OUT_FAST_T
#undef RET_OUT_FAST
    }
    if (wide)
        return fg_launch(retention_chunk_out_kernel<float>, dim3(n_chunks, H), dim3(RET_THREADS), s3, stream, proj, ld, (float *)out, ldo,
                         positions, (const int *)chunk_row, (const int *)chunk_len, cos_t, sin_t, decay, (const float *)U, H, dk, dv, k_scale, eps);
    return fg_launch(retention_chunk_out_kernel<bf16>, dim3(n_chunks, H), dim3(RET_THREADS), s3, stream, proj, ld, (bf16 *)out, ldo,
                     positions, (const int *)chunk_row, (const int *)chunk_len, cos_t, sin_t, decay, (const float *)U, H, dk, dv, k_scale, eps);
}
