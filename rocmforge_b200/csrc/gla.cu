// Gated linear attention: linear attention whose state decays by a factor of its own per key channel and per token,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (S is [dim, vdim] per (sequence, head)),
// with alpha_t = sigmoid(z_t)^(1/tau) from a projection z of the token.  Prompts (any number of tokens per sequence,
// continued from the state an earlier step left) and decoding (one token) run the same kernel.  Everything after the
// projections is 32-bit: q and k, the decay and its logarithm, the state, o.  The per-head norm and the gate that
// follow are retention's (retention_gate with a weight).
//
//   gla_prepare   q (times q_scale), k of the projection's row as float, and alpha = exp(log sigmoid(z) / tau) with
//                 log sigmoid(z) = min(z, 0) - log1p(exp(-|z|)): float [3, T, heads*dim]
//   gla_scan      the recurrence, token by token.  The state of a (sequence, head) is kept as [dim][vdim] (a row of S,
//                 one key channel, is contiguous).  A block owns (sequence, head, 32 value columns); the columns of S
//                 are independent of each other, so the blocks never talk.  A lane owns a column, a warp a slice of
//                 rows.  The order of every sum is fixed by (dim, position in the sequence) alone: how a prompt is cut
//                 into steps and what else is in the batch change no bit.
#include "common.cuh"

#define GL_TOK 16             // tokens staged in shared memory at a time
#define GL_SLICE 8            // rows of the state whose products with q are added up together: the unit of every kernel's sums

template <typename T>
__global__ void gla_prepare_kernel(const T* __restrict__ src, int row_stride, int q_col, int k_col,
                                   const float* __restrict__ z, float* __restrict__ qka, int width, float q_scale,
                                   float inv_tau, int T_) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)T_ * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width, c = idx - t * width;
        qka[idx] = Cvt<T>::to_f32(src[t * row_stride + q_col + c]) * q_scale;
        qka[n + idx] = Cvt<T>::to_f32(src[t * row_stride + k_col + c]);
        const float zz = z[idx];
        const float log_sig = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
        qka[2 * n + idx] = expf(log_sig * inv_tau);
    }
}

// grid (sequence, head, ceil(vdim / COLS)); the rows of the state are cut into slices of ROWS (8 or 16, by dim).  With COLS = 32 a warp
// holds one slice for the block's 32 value columns, lane l column j0 + l; with COLS = 16 (taken when the step has too few
// (sequence, head) pairs to give every SM a block of 32 columns) a warp holds two slices side by side for 16 columns.
// Either way a thread has ROWS state elements of one column in registers, and a column's arithmetic (slices of the
// same rows, added in the same order) is the same, so the choice changes no bit.
// Per token a thread updates its rows (s = alpha_i s + k_i v_j) and adds up s q_i over them (four partial sums, by
// i mod 4); q, k and alpha of the token's rows come from shared memory 16 bytes at a time, the same address for all
// lanes.  The warps' sums for the staged tokens go to shared memory and are added in warp order once per stage:
// no shuffles, one barrier pair per GL_TOK tokens, and a chain per token that is the state's FMA alone.
__device__ __forceinline__ void gl_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gl_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// One token for a thread's ROWS rows of one column: s <- a s + k v, and sum_r s q per slice of GL_SLICE rows (four partial
// sums by r mod 4 each).  The sums are formed slice by slice whatever ROWS is, so every kernel form gives the same bits.
template <int ROWS>
__device__ __forceinline__ void gl_token(float (&s)[ROWS], const float* __restrict__ a, const float* __restrict__ k,
                                         const float* __restrict__ q, float vj, float (&out)[ROWS / GL_SLICE]) {
#pragma unroll
    for (int u = 0; u < ROWS / GL_SLICE; ++u) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = u * GL_SLICE; r < (u + 1) * GL_SLICE; r += 4) {
            const float4 a4 = *reinterpret_cast<const float4*>(a + r);
            const float4 k4 = *reinterpret_cast<const float4*>(k + r);
            const float4 q4 = *reinterpret_cast<const float4*>(q + r);
            s[r + 0] = fmaf(a4.x, s[r + 0], k4.x * vj); acc[0] = fmaf(s[r + 0], q4.x, acc[0]);
            s[r + 1] = fmaf(a4.y, s[r + 1], k4.y * vj); acc[1] = fmaf(s[r + 1], q4.y, acc[1]);
            s[r + 2] = fmaf(a4.z, s[r + 2], k4.z * vj); acc[2] = fmaf(s[r + 2], q4.z, acc[2]);
            s[r + 3] = fmaf(a4.w, s[r + 3], k4.w * vj); acc[3] = fmaf(s[r + 3], q4.w, acc[3]);
        }
        out[u] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
}

// The same with ONE decay for all rows of the head (designs whose state decays by a scalar per head and token).
template <int ROWS>
__device__ __forceinline__ void gl_token_scalar(float (&s)[ROWS], float a, const float* __restrict__ k,
                                                const float* __restrict__ q, float vj, float (&out)[ROWS / GL_SLICE]) {
#pragma unroll
    for (int u = 0; u < ROWS / GL_SLICE; ++u) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = u * GL_SLICE; r < (u + 1) * GL_SLICE; r += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(k + r);
            const float4 q4 = *reinterpret_cast<const float4*>(q + r);
            s[r + 0] = fmaf(a, s[r + 0], k4.x * vj); acc[0] = fmaf(s[r + 0], q4.x, acc[0]);
            s[r + 1] = fmaf(a, s[r + 1], k4.y * vj); acc[1] = fmaf(s[r + 1], q4.y, acc[1]);
            s[r + 2] = fmaf(a, s[r + 2], k4.z * vj); acc[2] = fmaf(s[r + 2], q4.z, acc[2]);
            s[r + 3] = fmaf(a, s[r + 3], k4.w * vj); acc[3] = fmaf(s[r + 3], q4.w, acc[3]);
        }
        out[u] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
}

// SCALAR (the recurrence of designs with one decay a_t and one input scale b_t per head and token,
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,  o_t = S_t^T q_t):
// `alpha` is then float [T, heads, 2] = (a_t, b_t); q and k rows have `qk_stride` floats and hold qk_heads heads, head h
// reading head h / (heads / qk_heads) (several heads may share one q and k); with `nstate` the state has one more
// column, n_t = a_t n_(t-1) + b_t k_t (the column whose v is 1), kept as [slots, heads, dim], and its product with q goes
// to qn [T, heads].
// The tokens of a stage are copied into shared memory asynchronously while the stage before is computed (two buffers):
// with one sequence there are few blocks, and a block that waited for its loads between stages spent half its time so.
template <typename T, int COLS, int ROWS, bool SCALAR>
__global__ void __launch_bounds__(512)
gla_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ alpha,
                const T* __restrict__ v, int v_stride, float* __restrict__ state, float* __restrict__ o,
                const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, int dim, int vdim, int vec,
                int qk_heads, int qk_stride, float* __restrict__ nstate, float* __restrict__ qn) {
    extern __shared__ __align__(16) float sh[];
    constexpr int SPW = 32 / COLS;                    // row slices side by side in a warp
    const int slices = (blockDim.x >> 5) * SPW;
    const int dimP = slices * ROWS;                // dim rounded up to whole slices; the padding rows are zero
    const int buf = GL_TOK * dimP;
    float* qs = sh;                                   // q, k, alpha [2][GL_TOK][dimP] each
    float* ks = qs + 2 * buf;
    float* as = ks + 2 * buf;
    const int abuf = SCALAR ? 2 * GL_TOK : buf;       // one (a, b) pair a token instead of a decay per row
    float* vs = as + 2 * abuf;                        // v [2][GL_TOK][COLS]
    constexpr int PER = ROWS / GL_SLICE;              // slices of GL_SLICE rows in a thread's rows
    const int n_sl = slices * PER;
    float* part = vs + 2 * GL_TOK * COLS;             // the sums of the slices of GL_SLICE rows [GL_TOK][n_sl][COLS]
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = lane % COLS, slice = warp * SPW + lane / COLS;
    const int j = j0 + col, i0 = slice * ROWS;
    const int row0 = cu_q[b], row1 = cu_q[b + 1];
    const int slot = seq_slot[b];
    const int hq = SCALAR ? h / (heads / qk_heads) : h;
    const int width = SCALAR ? qk_stride : heads * dim;
    float* S = state + ((size_t)slot * heads + h) * dim * vdim;
    const bool has_n = SCALAR && nstate != nullptr;
    const bool ncol = has_n && j == vdim;             // this thread's column is the normaliser's
    float* Nn = has_n ? nstate + ((size_t)slot * heads + h) * dim : nullptr;
    // the padding rows never change: zero once, in both buffers
    for (int idx = threadIdx.x; idx < 2 * GL_TOK * (dimP - dim); idx += blockDim.x) {
        const int tt = idx / (dimP - dim), i = dim + idx - tt * (dimP - dim);
        qs[tt * dimP + i] = 0.f; ks[tt * dimP + i] = 0.f;
        if (!SCALAR) as[tt * dimP + i] = 0.f;
    }
    pdl_wait();
    float s[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
        s[r] = i0 + r < dim ? (j < vdim ? S[(size_t)(i0 + r) * vdim + j] : (ncol ? Nn[i0 + r] : 0.f)) : 0.f;

    // asynchronous copies of q, k, alpha of the stage that starts at token t0 into buffer p; the caller commits
    auto fetch = [&](int t0, int p) {
        const int cnt = min(GL_TOK, row1 - t0);
        if (vec) {
            const int d4 = dim >> 2;
            for (int idx = threadIdx.x; idx < cnt * d4; idx += blockDim.x) {
                const int tt = idx / d4, i = (idx - tt * d4) << 2;
                const size_t g = (size_t)(t0 + tt) * width + hq * dim + i;
                const int d = p * buf + tt * dimP + i;
                gl_copy16(qs + d, q + g); gl_copy16(ks + d, k + g);
                if (!SCALAR) gl_copy16(as + d, alpha + g);
            }
        } else {
            for (int idx = threadIdx.x; idx < cnt * dim; idx += blockDim.x) {
                const int tt = idx / dim, i = idx - tt * dim;
                const size_t g = (size_t)(t0 + tt) * width + hq * dim + i;
                const int d = p * buf + tt * dimP + i;
                gl_copy4(qs + d, q + g); gl_copy4(ks + d, k + g);
                if (!SCALAR) gl_copy4(as + d, alpha + g);
            }
        }
        if (SCALAR)
            for (int idx = threadIdx.x; idx < cnt * 2; idx += blockDim.x)
                gl_copy4(as + p * abuf + idx, alpha + ((size_t)(t0 + (idx >> 1)) * heads + h) * 2 + (idx & 1));
    };
    // v of a stage: GL_TOK * COLS values, up to sixteen per thread (a block has at least 32 threads), through registers
    auto v_value = [&](int t0, int idx) -> float {
        const int cnt = min(GL_TOK, row1 - t0);
        const int tt = idx / COLS, c = idx % COLS;
        if (tt < cnt && j0 + c < vdim) return Cvt<T>::to_f32(v[(size_t)(t0 + tt) * v_stride + h * vdim + j0 + c]);
        return (has_n && tt < cnt && j0 + c == vdim) ? 1.f : 0.f;
    };
    if (row0 < row1) {
        fetch(row0, 0);
        for (int idx = threadIdx.x; idx < GL_TOK * COLS; idx += blockDim.x) vs[idx] = v_value(row0, idx);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    int p = 0;
    for (int t0 = row0; t0 < row1; t0 += GL_TOK, p ^= 1) {
        const int cnt = min(GL_TOK, row1 - t0);
        const bool more = t0 + GL_TOK < row1;
        float v_next[16];                             // GL_TOK * COLS / 32 threads at least
        if (more) {
            fetch(t0 + GL_TOK, p ^ 1);
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int idx = threadIdx.x + u * blockDim.x;
                v_next[u] = idx < GL_TOK * COLS ? v_value(t0 + GL_TOK, idx) : 0.f;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");       // this stage's copies have landed (the next one's may fly)
        __syncthreads();
        const float* qb = qs + p * buf;
        const float* kb = ks + p * buf;
        const float* ab = as + p * abuf;
        const float* vb = vs + p * GL_TOK * COLS;
#pragma unroll 2
        for (int tt = 0; tt < cnt; ++tt) {
            float sums[PER];
            if constexpr (SCALAR)
                gl_token_scalar<ROWS>(s, ab[2 * tt], kb + tt * dimP + i0, qb + tt * dimP + i0, vb[tt * COLS + col] * ab[2 * tt + 1], sums);
            else
                gl_token<ROWS>(s, ab + tt * dimP + i0, kb + tt * dimP + i0, qb + tt * dimP + i0, vb[tt * COLS + col], sums);
#pragma unroll
            for (int u = 0; u < PER; ++u) part[(tt * n_sl + slice * PER + u) * COLS + col] = sums[u];
        }
        __syncthreads();                              // the sums are complete; this stage's buffers are used up
        for (int idx = threadIdx.x; idx < cnt * COLS; idx += blockDim.x) {
            const int tt = idx / COLS, c = idx % COLS;
            float sum = 0.f;
            for (int w = 0; w < n_sl; ++w) sum += part[(tt * n_sl + w) * COLS + c];
            if (j0 + c < vdim) o[(size_t)(t0 + tt) * heads * vdim + h * vdim + j0 + c] = sum;
            else if (has_n && qn != nullptr && j0 + c == vdim) qn[(size_t)(t0 + tt) * heads + h] = sum;
        }
        if (more) {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int idx = threadIdx.x + u * blockDim.x;
                if (idx < GL_TOK * COLS) vs[(p ^ 1) * GL_TOK * COLS + idx] = v_next[u];
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (j < vdim) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (i0 + r < dim) S[(size_t)(i0 + r) * vdim + j] = s[r];
    } else if (ncol) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (i0 + r < dim) Nn[i0 + r] = s[r];
    }
}

// One token per sequence (decoding): the same arithmetic without the staging.  grid (sequence, head, ceil(vdim / 32)),
// a warp per ROWS rows as above; a thread reads its rows' q, k and alpha straight from global memory (16 bytes at a
// time where aligned, the same address for all lanes of a warp) and its state elements once, and writes them once.
template <typename T, int ROWS, bool SCALAR>
__global__ void __launch_bounds__(512)
gla_decode_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ alpha,
                  const T* __restrict__ v, int v_stride, float* __restrict__ state, float* __restrict__ o,
                  const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, int dim, int vdim, int vec,
                  int qk_heads, int qk_stride, float* __restrict__ nstate, float* __restrict__ qn) {
    constexpr int PER = ROWS / GL_SLICE;
    __shared__ float part[32 * 32];                   // up to 256 / GL_SLICE slices
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int j = j0 + lane, i0 = warp * ROWS;
    const int t = cu_q[b];
    float* S = state + ((size_t)seq_slot[b] * heads + h) * dim * vdim;
    const bool ncol = SCALAR && nstate != nullptr && j == vdim;
    float* Nn = ncol ? nstate + ((size_t)seq_slot[b] * heads + h) * dim : nullptr;
    pdl_wait();
    float s[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
        s[r] = i0 + r < dim ? (j < vdim ? S[(size_t)(i0 + r) * vdim + j] : (ncol ? Nn[i0 + r] : 0.f)) : 0.f;
    const size_t g = SCALAR ? (size_t)t * qk_stride + (size_t)(h / (heads / qk_heads)) * dim + i0
                            : (size_t)t * heads * dim + (size_t)h * dim + i0;
    float a[ROWS], kk[ROWS], qq[ROWS];
    float bt = 1.f;
    if (SCALAR) {
        const float at = alpha[((size_t)t * heads + h) * 2];
        bt = alpha[((size_t)t * heads + h) * 2 + 1];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) a[r] = at;
    }
    if (vec && i0 + ROWS <= dim) {
#pragma unroll
        for (int r = 0; r < ROWS; r += 4) {
            if (!SCALAR) {
                const float4 a4 = *reinterpret_cast<const float4*>(alpha + g + r);
                a[r] = a4.x; a[r + 1] = a4.y; a[r + 2] = a4.z; a[r + 3] = a4.w;
            }
            const float4 k4 = *reinterpret_cast<const float4*>(k + g + r);
            const float4 q4 = *reinterpret_cast<const float4*>(q + g + r);
            kk[r] = k4.x; kk[r + 1] = k4.y; kk[r + 2] = k4.z; kk[r + 3] = k4.w;
            qq[r] = q4.x; qq[r + 1] = q4.y; qq[r + 2] = q4.z; qq[r + 3] = q4.w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const bool in = i0 + r < dim;
            if (!SCALAR) a[r] = in ? alpha[g + r] : 0.f;
            kk[r] = in ? k[g + r] : 0.f; qq[r] = in ? q[g + r] : 0.f;
        }
    }
    const float vj = (j < vdim ? Cvt<T>::to_f32(v[(size_t)t * v_stride + h * vdim + j]) : (ncol ? 1.f : 0.f)) * bt;
#pragma unroll
    for (int u = 0; u < PER; ++u) {                   // the same operations in the same order as gl_token
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = u * GL_SLICE; r < (u + 1) * GL_SLICE; ++r) {
            s[r] = fmaf(a[r], s[r], kk[r] * vj);
            acc[r & 3] = fmaf(s[r], qq[r], acc[r & 3]);
        }
        part[(warp * PER + u) * 32 + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    }
    if (j < vdim) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (i0 + r < dim) S[(size_t)(i0 + r) * vdim + j] = s[r];
    } else if (ncol) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (i0 + r < dim) Nn[i0 + r] = s[r];
    }
    __syncthreads();
    if (warp == 0 && (j < vdim || ncol)) {
        float sum = 0.f;
        for (int w = 0; w < warps * PER; ++w) sum += part[w * 32 + lane];
        if (j < vdim) o[(size_t)t * heads * vdim + h * vdim + j] = sum;
        else if (qn != nullptr) qn[(size_t)t * heads + h] = sum;
    }
}

// What the scalar form adds to a launch (all unused by the form with a decay per key channel).
struct ScalarArgs {
    int qk_heads, qk_stride;
    float* nstate;
    float* qn;
};

template <typename T, int COLS, int ROWS, bool SCALAR>
static int launch_scan_cols(const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                            float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int vec,
                            ScalarArgs x, cudaStream_t st) {
    constexpr int SPW = 32 / COLS;
    const int slices = ((dim + ROWS - 1) / ROWS + SPW - 1) / SPW * SPW;
    const int warps = slices / SPW;
    const int gz = (vdim + (x.nstate != nullptr ? 1 : 0) + COLS - 1) / COLS;
    if (gz > 65535) return RF_ERR_UNSUPPORTED;
    const size_t smem = (size_t)((SCALAR ? 4 : 6) * GL_TOK * slices * ROWS + (SCALAR ? 4 * GL_TOK : 0) + 2 * GL_TOK * COLS +
                                 GL_TOK * slices * (ROWS / GL_SLICE) * COLS) * sizeof(float);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<T, COLS, ROWS, SCALAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    rf_launch(gla_scan_kernel<T, COLS, ROWS, SCALAR>, dim3(B, heads, gz), dim3(warps * 32), smem, st, q, k, alpha, reinterpret_cast<const T*>(v),
              v_stride, state, o, cu_q, seq_slot, heads, dim, vdim, vec, x.qk_heads, x.qk_stride, x.nstate, x.qn);
    RF_LAUNCH_CHECK();
    return 0;
}

// ROWS: the rows of the state in a thread's registers (see launch_scan).
template <typename T, int ROWS, bool SCALAR>
static int launch_scan_rows(const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                            float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int one_token,
                            int sms, ScalarArgs x, cudaStream_t st) {
    const int warps = (dim + ROWS - 1) / ROWS;
    const int cols = vdim + (x.nstate != nullptr ? 1 : 0);
    const int gz = (cols + 31) / 32;
    if (warps > 16 || gz > 65535) return RF_ERR_UNSUPPORTED;
    // rows of q, k, alpha are copied 16 bytes at a time where a head's slice of every token starts on such a boundary
    const int vec = dim % 4 == 0 && (!SCALAR || x.qk_stride % 4 == 0) &&
                    !((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                       (SCALAR ? 0 : reinterpret_cast<uintptr_t>(alpha))) & 15);
    if (one_token) {
        rf_launch(gla_decode_kernel<T, ROWS, SCALAR>, dim3(B, heads, gz), dim3(warps * 32), 0, st, q, k, alpha, reinterpret_cast<const T*>(v),
                  v_stride, state, o, cu_q, seq_slot, heads, dim, vdim, vec, x.qk_heads, x.qk_stride, x.nstate, x.qn);
        RF_LAUNCH_CHECK();
        return 0;
    }
    if (sms <= 0) sms = 148;
    if ((long long)B * heads * gz < sms)              // few blocks: narrower ones, twice as many
        return launch_scan_cols<T, 16, ROWS, SCALAR>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, vec, x, st);
    return launch_scan_cols<T, 32, ROWS, SCALAR>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, vec, x, st);
}

template <typename T, bool SCALAR>
static int launch_scan(const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                       float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int one_token,
                       int sms, ScalarArgs x, cudaStream_t st) {
    if (B <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || heads <= 0 || heads > 65535) return RF_ERR_UNSUPPORTED;
    if (SCALAR && (x.qk_heads <= 0 || heads % x.qk_heads || x.qk_stride < x.qk_heads * dim)) return RF_ERR_BAD_ARG;
    // Eight rows a thread (twice the warps, half the chain of each) while the step has too few (sequence, head) pairs to
    // fill the SMs twice over, sixteen beyond (fewer instructions per product) and for more than 128 key channels (a block
    // has at most sixteen warps).  Measured on 16 heads of 128 x 128, 2,048 tokens a sequence: one sequence 533 us with
    // sixteen rows, 434 us with eight; eight sequences 1,700 against 2,518 us.  The sums are formed per slice of GL_SLICE
    // rows in both, so the choice changes no bit.
    if (sms <= 0) sms = 148;
    if (dim <= 128 && (long long)B * heads * ((vdim + 31) / 32) < 2LL * sms)
        return launch_scan_rows<T, 8, SCALAR>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, one_token, sms, x, st);
    return launch_scan_rows<T, 16, SCALAR>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, one_token, sms, x, st);
}

template <typename T>
static int launch_prepare(const void* src, int row_stride, int q_col, int k_col, const float* z, float* qka, int width,
                          float q_scale, float tau, int T_, cudaStream_t st) {
    const size_t n = (size_t)T_ * width;
    if (n == 0) return 0;
    if (!(tau > 0.f)) return RF_ERR_BAD_ARG;
    const size_t blocks = (n + 255) / 256;
    rf_launch(gla_prepare_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st,
              reinterpret_cast<const T*>(src), row_stride, q_col, k_col, z, qka, width, q_scale, 1.f / tau, T_);
    RF_LAUNCH_CHECK();
    return 0;
}

// dtype: 0 = float32, 1 = bfloat16 (of the projection's output and of v)
extern "C" {
// src [T, row_stride]: q at columns q_col.., k at k_col.. (width = heads*dim each); z float [T, width]; qka float [3, T, width]
int rf_gla_prepare(int dtype, const void* src, int row_stride, int q_col, int k_col, const float* z, float* qka, int width,
                   float q_scale, float tau, int T_, cudaStream_t st) {
    return dtype == 0 ? launch_prepare<float>(src, row_stride, q_col, k_col, z, qka, width, q_scale, tau, T_, st)
                      : launch_prepare<__nv_bfloat16>(src, row_stride, q_col, k_col, z, qka, width, q_scale, tau, T_, st);
}
// state float [slots, heads, dim, vdim]; o float [T, heads*vdim]; one_token: every sequence of the step brings exactly
// one token (the kernel without staging; the same bits as the general one)
// sms: multiprocessors of the device (sizes the blocks)
int rf_gla_scan(int dtype, const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int one_token, int sms,
                cudaStream_t st) {
    const ScalarArgs none = {heads, heads * dim, nullptr, nullptr};
    return dtype == 0 ? launch_scan<float, false>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, one_token, sms, none, st)
                      : launch_scan<__nv_bfloat16, false>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, one_token, sms, none, st);
}
// The recurrence with one decay and one input scale per head and token: S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t.
// q, k float rows of qk_stride floats that hold qk_heads heads of dim (head h reads head h / (heads / qk_heads));
// ab float [T, heads, 2] = (a_t, b_t); v [T, v_stride] of dtype (heads * vdim columns); state float [slots, heads, dim, vdim].
// nstate (may be null) float [slots, heads, dim]: n_t = a_t n_(t-1) + b_t k_t, and qn float [T, heads] receives n_t . q_t.
int rf_gated_scan(int dtype, const float* q, const float* k, int qk_heads, int qk_stride, const float* ab, const void* v,
                  int v_stride, float* state, float* nstate, float* o, float* qn, const int* cu_q, const int* seq_slot, int B,
                  int heads, int dim, int vdim, int one_token, int sms, cudaStream_t st) {
    const ScalarArgs x = {qk_heads, qk_stride, nstate, qn};
    return dtype == 0 ? launch_scan<float, true>(q, k, ab, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, one_token, sms, x, st)
                      : launch_scan<__nv_bfloat16, true>(q, k, ab, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, one_token, sms, x, st);
}
}
