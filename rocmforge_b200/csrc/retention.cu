// Retention: linear attention with a fixed decay per head and a matrix state per (sequence, head),
//   S_t = decay_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
// for prompts (any number of tokens per sequence, continued from the state an earlier step left) and for
// decoding (one token), by the same kernels.  Everything after the projections is 32-bit: the rotation's angle,
// q and k after rotation, the state, o, its per-head unit norm.
//
//   retention_prepare   q, k of the projection's row -> rotated (first rot_dim elements of a head, pairs
//                       (i, i + rot_dim/2), angle float(pos) * inv_freq[i]), k scaled, as float [2, T, heads*dim]
//   The state of a (sequence, head) is kept as [vdim][dim]: a column of S (one value dimension) is contiguous, so a
//   warp that owns a column reads and writes whole 128-byte lines.
//   retention_scan      the recurrence, token by token: a block owns (sequence, head, a slice of 8 value columns);
//                       the columns of S are independent of each other, so the slices never talk.  A warp owns one
//                       column; a lane holds the rows lane, lane + 32, ... of it in registers.  The order of every sum
//                       is fixed by (dim, position in the sequence) alone: how a prompt is cut into steps, or what
//                       else is in the batch, changes no bit.
//   retention_gate      o / rms(o) per head, times silu(gate), into the compute dtype for the output product
#include "common.cuh"

#define RT_COLS 8             // value columns (warps) of a scan block
#define RT_TOK 16             // tokens staged in shared memory at a time

// A thread per unit of a head: a rotated pair (elements e and e + rot_dim/2 of q and of k: one sine and cosine serve all
// four), or an element beyond the rotated ones.
template <typename T>
__global__ void retention_prepare_kernel(const T* __restrict__ src, int row_stride, int q_col, int k_col,
                                         float* __restrict__ qk, int heads, int dim, int rot_dim,
                                         const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                         float k_scale, int T_) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int width = heads * dim;
    const int pos = tok_pos[t];
    const int rh = rot_dim >> 1;
    const int units = rh + (dim - rot_dim);               // per head
    pdl_wait();
    const T* qrow = src + (size_t)t * row_stride + q_col;
    const T* krow = src + (size_t)t * row_stride + k_col;
    float* qo = qk + (size_t)t * width;
    float* ko = qk + (size_t)T_ * width + (size_t)t * width;
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < heads * units; idx += gridDim.y * blockDim.x) {
        const int h = idx / units, u = idx - h * units;
        if (u < rh) {
            const int c0 = h * dim + u, c1 = c0 + rh;
            float sn, cs;
            sincosf((float)pos * inv_freq[u], &sn, &cs);
            const float q0 = Cvt<T>::to_f32(qrow[c0]), q1 = Cvt<T>::to_f32(qrow[c1]);
            const float k0 = Cvt<T>::to_f32(krow[c0]), k1 = Cvt<T>::to_f32(krow[c1]);
            qo[c0] = q0 * cs - q1 * sn;
            qo[c1] = q1 * cs + q0 * sn;
            ko[c0] = (k0 * cs - k1 * sn) * k_scale;
            ko[c1] = (k1 * cs + k0 * sn) * k_scale;
        } else {
            const int c = h * dim + rot_dim + (u - rh);
            qo[c] = Cvt<T>::to_f32(qrow[c]);
            ko[c] = Cvt<T>::to_f32(krow[c]) * k_scale;
        }
    }
}

// grid (sequence, head, ceil(vdim / RT_COLS)); block RT_COLS warps.  R = ceil(dim / 32) rows of a column per lane.
template <typename T, int R>
__global__ void __launch_bounds__(RT_COLS * 32)
retention_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const T* __restrict__ v, int v_stride,
                      float* __restrict__ state, const float* __restrict__ decay, float* __restrict__ o,
                      const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
    extern __shared__ float sh[];                     // q [RT_TOK][dim], k [RT_TOK][dim], v [RT_TOK][RT_COLS]
    float* qs = sh;
    float* ks = qs + RT_TOK * dim;
    float* vs = ks + RT_TOK * dim;
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * RT_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = j0 + warp;
    const int row0 = cu_q[b], row1 = cu_q[b + 1];
    const int slot = seq_slot[b];
    const float d = decay[h];
    const int width = heads * dim;
    float* S = state + (((size_t)slot * heads + h) * vdim + (j < vdim ? j : 0)) * dim;      // this warp's column
    pdl_wait();
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        s[r] = (i < dim && j < vdim) ? S[i] : 0.f;
    }
    for (int t0 = row0; t0 < row1; t0 += RT_TOK) {
        const int cnt = min(RT_TOK, row1 - t0);
        __syncthreads();                              // the tokens before are used up
        for (int idx = threadIdx.x; idx < cnt * dim; idx += blockDim.x) {
            const int tt = idx / dim, i = idx - tt * dim;
            qs[idx] = q[(size_t)(t0 + tt) * width + h * dim + i];
            ks[idx] = k[(size_t)(t0 + tt) * width + h * dim + i];
        }
        for (int idx = threadIdx.x; idx < cnt * RT_COLS; idx += blockDim.x) {
            const int tt = idx / RT_COLS, c = idx - tt * RT_COLS;
            vs[idx] = (j0 + c < vdim) ? Cvt<T>::to_f32(v[(size_t)(t0 + tt) * v_stride + h * vdim + j0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < cnt; ++tt) {
            const float vj = vs[tt * RT_COLS + warp];
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = lane + 32 * r;
                if (i < dim) {
                    s[r] = fmaf(d, s[r], ks[tt * dim + i] * vj);
                    acc = fmaf(s[r], qs[tt * dim + i], acc);
                }
            }
            acc = warp_sum(acc);
            if (lane == 0 && j < vdim) o[(size_t)(t0 + tt) * heads * vdim + h * vdim + j] = acc;
        }
    }
    if (j < vdim) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = lane + 32 * r;
            if (i < dim) S[i] = s[r];
        }
    }
}

// a warp per (token, head): out = o / sqrt(mean(o^2) + eps) (* w, a weight [vdim] shared by the heads, if given) * silu(gate)
template <typename T>
__global__ void retention_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                                      T* __restrict__ out, int heads, int vdim, float eps, int T_,
                                      const void* __restrict__ norm_w, int w_is_f32, int w_per_head, int sigmoid,
                                      const float* __restrict__ qn, const float* __restrict__ mt) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long total = (long long)T_ * heads;
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
         w += (long long)gridDim.x * (blockDim.x >> 5)) {
        const long long t = w / heads;
        const int h = (int)(w - t * heads);
        const float* orow = o + (size_t)t * heads * vdim + (size_t)h * vdim;
        // a denominator of the head: max(|n . q|, exp(-m)) + 1e-6, before the norm (designs with a normaliser state)
        const float inv = qn != nullptr ? 1.f / (fmaxf(fabsf(qn[w]), expf(-mt[w])) + 1e-6f) : 1.f;
        float ss = 0.f;
        for (int e = lane; e < vdim; e += 32) { const float x = orow[e] * inv; ss += x * x; }
        const float r = rsqrtf(warp_sum(ss) / (float)vdim + eps);
        for (int e = lane; e < vdim; e += 32) {
            const float g = Cvt<T>::to_f32(gate[(size_t)t * gate_stride + (size_t)h * vdim + e]);
            const float wn = norm_w != nullptr ? load_vec(norm_w, w_is_f32, w_per_head ? h * vdim + e : e) : 1.f;
            const float gv = sigmoid ? 1.f / (1.f + expf(-g)) : g / (1.f + expf(-g));
            out[(size_t)t * heads * vdim + (size_t)h * vdim + e] = Cvt<T>::from_f32(orow[e] * inv * r * wn * gv);
        }
    }
}

// ---------------------------------------------------------------- prompts: the recurrence in chunks of 64 tokens
// The same sums in another order, so that a prompt's chunks run side by side instead of token after token.  With
// positions t, s inside a chunk of cnt tokens, S0 the state before the chunk and d the head's decay:
//   pass 1 (chunks side by side)   L = sum_s d^(cnt-1-s) k_s v_s^T                              [dim, vdim]
//   pass 2 (chunk after chunk, element by element)   S0 of every chunk; the state after the last one
//                                   S0(next) = d^cnt S0 + L      (L's place in memory becomes S0's)
//   pass 3 (chunks side by side)   o_t = sum_(s<=t) d^(t-s) (q_t . k_s) v_s + d^(t+1) S0^T q_t
// All in 32-bit on the CUDA cores (the scores of this mixer are not rounded to 16 bits).  The chunk table is built on
// the host with the step: first[B+1] (index of each sequence's first chunk), then (sequence, first row) per chunk.
#define RC 64                 // tokens of a chunk
#define RC_LD 68              // row stride of the transposed tiles: rows stay 16-byte aligned
#define RV 64                 // value columns of a block

// grid (chunk, head, ceil(vdim / RV)); 256 threads: thread (ty, tx) owns rows ty * RPT .. + RPT - 1 (RPT = 4, 8, 12 or 16
// by dim) and columns 4 tx .. 4 tx + 3: per key, 16-byte loads of its k rows and of its v columns feed 4 RPT FMAs
template <typename T>
__global__ void __launch_bounds__(256)
retention_chunk_state_kernel(const float* __restrict__ k, const T* __restrict__ v, int v_stride, float* __restrict__ LS,
                             const float* __restrict__ decay, const int* __restrict__ table, const int* __restrict__ cu_q,
                             int B, int heads, int dim, int vdim) {
    extern __shared__ __align__(16) float sh[];
    const int dimP = (dim + 3) & ~3;                  // rows of 16-byte groups
    float* ks = sh;                                   // [RC][dimP], already times d^(cnt-1-s)
    float* vs = ks + RC * dimP;                       // [RC][RV]
    float* pw = vs + RC * RV;                         // d^0 .. d^(RC-1)
    pdl_trigger();
    const int c = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * RV;
    const int b = table[B + 1 + 2 * c], q0 = table[B + 2 + 2 * c];
    const int row0 = cu_q[b] + q0, cnt = min(RC, cu_q[b + 1] - row0);
    const int width = heads * dim;
    if (threadIdx.x < RC) pw[threadIdx.x] = powf(decay[h], (float)threadIdx.x);
    pdl_wait();
    __syncthreads();
    for (int idx = threadIdx.x; idx < cnt * dimP; idx += 256) {
        const int s = idx / dimP, i = idx - s * dimP;
        ks[idx] = i < dim ? k[(size_t)(row0 + s) * width + h * dim + i] * pw[cnt - 1 - s] : 0.f;
    }
    for (int idx = threadIdx.x; idx < cnt * RV; idx += 256) {
        const int s = idx / RV, j = idx - s * RV;
        vs[idx] = (j0 + j < vdim) ? Cvt<T>::to_f32(v[(size_t)(row0 + s) * v_stride + h * vdim + j0 + j]) : 0.f;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int groups = (dim + 63) / 64;               // 16-byte groups of rows per thread
    const int i0 = ty * 4 * groups;
    float acc[16][4];
#pragma unroll
    for (int r = 0; r < 16; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
    for (int s = 0; s < cnt; ++s) {
        const float4 vv = *reinterpret_cast<const float4*>(&vs[s * RV + 4 * tx]);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if (g < groups && i0 + 4 * g < dimP) {
                const float4 kk = *reinterpret_cast<const float4*>(&ks[s * dimP + i0 + 4 * g]);
                const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    acc[4 * g + x][0] = fmaf(kv[x], vv.x, acc[4 * g + x][0]); acc[4 * g + x][1] = fmaf(kv[x], vv.y, acc[4 * g + x][1]);
                    acc[4 * g + x][2] = fmaf(kv[x], vv.z, acc[4 * g + x][2]); acc[4 * g + x][3] = fmaf(kv[x], vv.w, acc[4 * g + x][3]);
                }
            }
        }
    }
    float* out = LS + (((size_t)c * heads + h) * dim) * vdim;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        const int i = i0 + r;
        if (r < 4 * groups && i < dim)
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (j0 + 4 * tx + u < vdim) out[(size_t)i * vdim + j0 + 4 * tx + u] = acc[r][u];
    }
}

// grid (sequence, head, blocks over dim * vdim); a thread owns one element of the state through all chunks
__global__ void __launch_bounds__(256)
retention_chunk_carry_kernel(float* __restrict__ LS, float* __restrict__ state, const float* __restrict__ decay,
                                             const int* __restrict__ table, const int* __restrict__ cu_q,
                                             const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= dim * vdim) return;
    const int c0 = table[b], c1 = table[b + 1];
    const int n_new = cu_q[b + 1] - cu_q[b];
    const float d = decay[h];
    const float d_full = powf(d, (float)RC);
    float* S = state + (((size_t)seq_slot[b] * heads + h) * vdim + e % vdim) * dim + e / vdim;     // kept as [vdim][dim]
    pdl_wait();
    float s = *S;
    const size_t step = (size_t)heads * dim * vdim;
    float* p = LS + (((size_t)c0 * heads + h) * dim) * vdim + e;
    for (int c = c0; c < c1; c += 8) {                   // eight chunks' sums on their way at once; the chain is the FMAs alone
        float l[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) l[u] = (c + u < c1) ? p[(size_t)u * step] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (c + u < c1) {
                p[(size_t)u * step] = s;                 // the state before chunk c + u
                const int cnt = min(RC, n_new - (c + u - c0) * RC);
                s = fmaf(cnt == RC ? d_full : powf(d, (float)cnt), s, l[u]);
            }
        p += 8 * step;
    }
    *S = s;
}

// grid (chunk, head, ceil(vdim / RV)); 256 threads as a 16 x 16 grid of 4 x 4 tiles
template <typename T>
__global__ void __launch_bounds__(256)
retention_chunk_out_kernel(const float* __restrict__ q, const float* __restrict__ k, const T* __restrict__ v, int v_stride,
                           const float* __restrict__ LS, const float* __restrict__ decay, float* __restrict__ o,
                           const int* __restrict__ table, const int* __restrict__ cu_q, int B, int heads, int dim, int vdim) {
    extern __shared__ __align__(16) float sh[];
    float* qt = sh;                                   // [dim][RC_LD]: q transposed
    float* kt = qt + dim * RC_LD;                     // [dim][RC_LD]: k transposed; later the state S0 as [dim][RV]
    float* vs = kt + dim * RC_LD;                     // [RC][RV]
    float* at = vs + RC * RV;                         // [RC (s)][RC_LD (t)]: the decayed scores, transposed
    float* pw = at + RC * RC_LD;                      // d^0 .. d^RC
    pdl_trigger();
    const int c = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * RV;
    const int b = table[B + 1 + 2 * c], q0 = table[B + 2 + 2 * c];
    const int row0 = cu_q[b] + q0, cnt = min(RC, cu_q[b + 1] - row0);
    const float d = decay[h];
    const int width = heads * dim;
    if (threadIdx.x <= RC) pw[threadIdx.x] = powf(d, (float)threadIdx.x);
    pdl_wait();
    for (int idx = threadIdx.x; idx < RC * dim; idx += 256) {
        const int s = idx / dim, i = idx - s * dim;
        const bool in = s < cnt;
        qt[i * RC_LD + s] = in ? q[(size_t)(row0 + s) * width + h * dim + i] : 0.f;
        kt[i * RC_LD + s] = in ? k[(size_t)(row0 + s) * width + h * dim + i] : 0.f;
    }
    for (int idx = threadIdx.x; idx < RC * RV; idx += 256) {
        const int s = idx / RV, j = idx - s * RV;
        vs[idx] = (s < cnt && j0 + j < vdim) ? Cvt<T>::to_f32(v[(size_t)(row0 + s) * v_stride + h * vdim + j0 + j]) : 0.f;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;        // rows (t) 4 ty .., columns 4 tx ..
    {
        // scores: a[t][s] = (q_t . k_s) d^(t-s) for s <= t
        float a[4][4];
#pragma unroll
        for (int x = 0; x < 4; ++x) { a[x][0] = a[x][1] = a[x][2] = a[x][3] = 0.f; }
        if (tx <= ty) {                                  // tiles above the diagonal are zero
            for (int i = 0; i < dim; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(&qt[i * RC_LD + 4 * ty]);
                const float4 kk = *reinterpret_cast<const float4*>(&kt[i * RC_LD + 4 * tx]);
                const float qv[4] = {qq.x, qq.y, qq.z, qq.w}, kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) a[x][y] = fmaf(qv[x], kv[y], a[x][y]);
            }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                const int t = 4 * ty + x, s = 4 * tx + y;
                at[s * RC_LD + t] = (s <= t) ? a[x][y] * pw[t - s] : 0.f;
            }
    }
    __syncthreads();                                     // k is used up: its place takes the state before the chunk
    const float* S0 = LS + (((size_t)c * heads + h) * dim) * vdim;
    for (int idx = threadIdx.x; idx < dim * RV; idx += 256) {
        const int i = idx / RV, j = idx - i * RV;
        kt[idx] = (j0 + j < vdim) ? S0[(size_t)i * vdim + j0 + j] : 0.f;
    }
    __syncthreads();
    float o1[4][4], o2[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) { o1[x][y] = 0.f; o2[x][y] = 0.f; }
    const int s_end = min(cnt, 4 * ty + 4);              // later keys have zero scores for these rows
    for (int s = 0; s < s_end; ++s) {
        const float4 aa = *reinterpret_cast<const float4*>(&at[s * RC_LD + 4 * ty]);
        const float4 vv = *reinterpret_cast<const float4*>(&vs[s * RV + 4 * tx]);
        const float av[4] = {aa.x, aa.y, aa.z, aa.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) o1[x][y] = fmaf(av[x], vw[y], o1[x][y]);
    }
    for (int i = 0; i < dim; ++i) {
        const float4 qq = *reinterpret_cast<const float4*>(&qt[i * RC_LD + 4 * ty]);
        const float4 ss = *reinterpret_cast<const float4*>(&kt[i * RV + 4 * tx]);
        const float qv[4] = {qq.x, qq.y, qq.z, qq.w}, sv[4] = {ss.x, ss.y, ss.z, ss.w};
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) o2[x][y] = fmaf(qv[x], sv[y], o2[x][y]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        const int t = 4 * ty + x;
        if (t < cnt)
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                const int j = j0 + 4 * tx + y;
                if (j < vdim) o[(size_t)(row0 + t) * heads * vdim + h * vdim + j] = fmaf(pw[t + 1], o2[x][y], o1[x][y]);
            }
    }
}

template <typename T>
static int launch_chunked(const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                          float* o, float* LS, const int* table, int n_chunks, const int* cu_q, const int* seq_slot, int B,
                          int heads, int dim, int vdim, cudaStream_t st) {
    if (B <= 0 || n_chunks <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || heads <= 0 || heads > 65535 || B > 65535) return RF_ERR_UNSUPPORTED;
    const int vz = (vdim + RV - 1) / RV;
    const size_t smem1 = (size_t)(RC * ((dim + 3) & ~3) + RC * RV + RC) * sizeof(float);
    const size_t smem3 = (size_t)(2 * dim * RC_LD + RC * RV + RC * RC_LD + RC + 4) * sizeof(float);
    static size_t set1 = 48 * 1024, set3 = 48 * 1024;
    if (smem1 > set1) {
        cudaError_t e = cudaFuncSetAttribute(retention_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (e != cudaSuccess) return (int)e;
        set1 = smem1;
    }
    if (smem3 > set3) {
        cudaError_t e = cudaFuncSetAttribute(retention_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
        if (e != cudaSuccess) return (int)e;
        set3 = smem3;
    }
    rf_launch(retention_chunk_state_kernel<T>, dim3(n_chunks, heads, vz), dim3(256), smem1, st, k, reinterpret_cast<const T*>(v),
              v_stride, LS, decay, table, cu_q, B, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    rf_launch(retention_chunk_carry_kernel, dim3(B, heads, (dim * vdim + 255) / 256), dim3(256), 0, st, LS, state, decay, table,
              cu_q, seq_slot, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    rf_launch(retention_chunk_out_kernel<T>, dim3(n_chunks, heads, vz), dim3(256), smem3, st, q, k, reinterpret_cast<const T*>(v),
              v_stride, (const float*)LS, decay, o, table, cu_q, B, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_prepare(const void* src, int row_stride, int q_col, int k_col, float* qk, int heads, int dim,
                          int rot_dim, const float* inv_freq, const int* tok_pos, float k_scale, int T_, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (rot_dim < 0 || rot_dim % 2 || rot_dim > dim) return RF_ERR_BAD_ARG;
    // few tokens: a row's elements over several blocks, so that the sines and cosines of a row do not queue in one
    int by = T_ >= 512 ? 1 : (heads * dim + 255) / 256;
    if (by > 64) by = 64;
    rf_launch(retention_prepare_kernel<T>, dim3(T_, by), dim3(256), 0, st, reinterpret_cast<const T*>(src), row_stride, q_col, k_col,
              qk, heads, dim, rot_dim, inv_freq, tok_pos, k_scale, T_);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T, int R>
static int launch_scan_r(const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                         float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    const size_t smem = (size_t)(2 * RT_TOK * dim + RT_TOK * RT_COLS) * sizeof(float);
    dim3 grid(B, heads, (vdim + RT_COLS - 1) / RT_COLS);
    rf_launch(retention_scan_kernel<T, R>, grid, dim3(RT_COLS * 32), smem, st, q, k, reinterpret_cast<const T*>(v), v_stride, state,
              decay, o, cu_q, seq_slot, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_scan(const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                       float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    if (B <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || heads <= 0 || heads > 65535 || (vdim + RT_COLS - 1) / RT_COLS > 65535)
        return RF_ERR_UNSUPPORTED;
    switch ((dim + 31) / 32) {
        case 1: return launch_scan_r<T, 1>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 2: return launch_scan_r<T, 2>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 3: return launch_scan_r<T, 3>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 4: return launch_scan_r<T, 4>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 5: case 6: return launch_scan_r<T, 6>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        default: return launch_scan_r<T, 8>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
    }
}

template <typename T>
static int launch_gate(const float* o, const void* gate, int gate_stride, void* out, int heads, int vdim, float eps, int T_,
                       cudaStream_t st, const void* w = nullptr, int w_is_f32 = 0, int w_per_head = 0, int sigmoid = 0,
                       const float* qn = nullptr, const float* mt = nullptr) {
    const long long total = (long long)T_ * heads;
    if (total <= 0) return 0;
    const long long blocks = (total + 7) / 8;
    rf_launch(retention_gate_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st, o,
              reinterpret_cast<const T*>(gate), gate_stride, reinterpret_cast<T*>(out), heads, vdim, eps, T_, w, w_is_f32, w_per_head,
              sigmoid, qn, mt);
    RF_LAUNCH_CHECK();
    return 0;
}

// dtype: 0 = float32, 1 = bfloat16 (of the projection's output, of v, of the gate and of the gated result)
extern "C" {
int rf_retention_prepare(int dtype, const void* src, int row_stride, int q_col, int k_col, float* qk, int heads, int dim,
                         int rot_dim, const float* inv_freq, const int* tok_pos, float k_scale, int T_, cudaStream_t st) {
    return dtype == 0 ? launch_prepare<float>(src, row_stride, q_col, k_col, qk, heads, dim, rot_dim, inv_freq, tok_pos, k_scale, T_, st)
                      : launch_prepare<__nv_bfloat16>(src, row_stride, q_col, k_col, qk, heads, dim, rot_dim, inv_freq, tok_pos, k_scale, T_, st);
}
int rf_retention_scan(int dtype, const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                      float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    return dtype == 0 ? launch_scan<float>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st)
                      : launch_scan<__nv_bfloat16>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
}
// The recurrence of a prompt step in chunks of 64 tokens (see above).  LS: scratch float [n_chunks, heads, dim, vdim];
// table: first[B+1], then n_chunks pairs (sequence, first row of the chunk among the sequence's new tokens).
int rf_retention_chunked(int dtype, const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                         float* o, float* LS, const int* table, int n_chunks, const int* cu_q, const int* seq_slot, int B,
                         int heads, int dim, int vdim, cudaStream_t st) {
    return dtype == 0 ? launch_chunked<float>(q, k, v, v_stride, state, decay, o, LS, table, n_chunks, cu_q, seq_slot, B, heads, dim, vdim, st)
                      : launch_chunked<__nv_bfloat16>(q, k, v, v_stride, state, decay, o, LS, table, n_chunks, cu_q, seq_slot, B, heads, dim, vdim, st);
}
int rf_retention_gate(int dtype, const float* o, const void* gate, int gate_stride, void* out, int heads, int vdim, float eps,
                      int T_, cudaStream_t st) {
    return dtype == 0 ? launch_gate<float>(o, gate, gate_stride, out, heads, vdim, eps, T_, st)
                      : launch_gate<__nv_bfloat16>(o, gate, gate_stride, out, heads, vdim, eps, T_, st);
}
// The same with a weight [vdim] of the per-head norm, shared by the heads.
int rf_retention_gate_w(int dtype, const float* o, const void* gate, int gate_stride, void* out, int heads, int vdim, float eps,
                        int T_, const void* w, int w_is_f32, cudaStream_t st) {
    return dtype == 0 ? launch_gate<float>(o, gate, gate_stride, out, heads, vdim, eps, T_, st, w, w_is_f32)
                      : launch_gate<__nv_bfloat16>(o, gate, gate_stride, out, heads, vdim, eps, T_, st, w, w_is_f32);
}
// The general form: the weight is [vdim] for all heads or (w_per_head) [heads * vdim]; the gate's function is silu or
// (sigmoid) the sigmoid; with qn and mt (float [T, heads] each) every head is first divided by
// max(|qn|, exp(-mt)) + 1e-6.
int rf_retention_gate_x(int dtype, const float* o, const void* gate, int gate_stride, void* out, int heads, int vdim, float eps,
                        int T_, const void* w, int w_is_f32, int w_per_head, int sigmoid, const float* qn, const float* mt,
                        cudaStream_t st) {
    if ((qn == nullptr) != (mt == nullptr)) return RF_ERR_BAD_ARG;
    return dtype == 0 ? launch_gate<float>(o, gate, gate_stride, out, heads, vdim, eps, T_, st, w, w_is_f32, w_per_head, sigmoid, qn, mt)
                      : launch_gate<__nv_bfloat16>(o, gate, gate_stride, out, heads, vdim, eps, T_, st, w, w_is_f32, w_per_head, sigmoid, qn, mt);
}
}
