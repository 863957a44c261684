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
// ---------------------------------------------------------------- prompts: the scalar form in chunks of 64 tokens
// S_t = a_t S_(t-1) + b_t k_t v_t^T with one (a_t, b_t) per head and token: the same sums in another order, so that a prompt's
// chunks run side by side instead of token after token.  With t, s inside a chunk of cnt tokens, S0 the state before it,
// P_t = a_0 ... a_t and w(t, s) = b_s a_(s+1) ... a_t (running products, formed by multiplying on: no logarithm and no
// quotient, so a decay of exactly 0 or 1 is like any other):
//   pass 1 (chunks side by side)   L = sum_s w(cnt-1, s) k_s v_s^T   [dim, vdim],  the same sum without v for the
//                                   normaliser, and the chunk's whole decay P_(cnt-1)
//   pass 2 (chunk after chunk, element by element)   S0(next) = P_(cnt-1) S0 + L      (L's place in memory becomes S0's)
//   pass 3 (chunks side by side)   o_t = sum_(s<=t) w(t, s) (q_t . k_s) v_s + P_t S0^T q_t, and for the normaliser
//                                   n_t . q_t = sum_(s<=t) w(t, s) (q_t . k_s) + P_t n0 . q_t
// All 32-bit on the CUDA cores.  The chunk table is retention's: first[B+1], then (sequence, first row) per chunk.
// Differs from the scan by rounding only.
#define GC 64                 // tokens of a chunk
#define GC_LD 68              // row stride of the transposed tiles: rows stay 16-byte aligned
#define GV 64                 // value columns of a block

// grid (chunk, head, ceil(vdim / GV)); 256 threads: thread (ty, tx) owns rows ty * RPT .. + RPT - 1 (RPT = 4, 8, 12 or 16
// by dim) and columns 4 tx .. 4 tx + 3 of L
template <typename T>
__global__ void __launch_bounds__(256)
gated_chunk_state_kernel(const float* __restrict__ k, int qk_heads, int qk_stride, const float* __restrict__ ab,
                         const T* __restrict__ v, int v_stride, float* __restrict__ LS, float* __restrict__ NL,
                         float* __restrict__ CD, const int* __restrict__ table, const int* __restrict__ cu_q, int B,
                         int heads, int dim, int vdim) {
    extern __shared__ __align__(16) float sh[];
    const int dimP = (dim + 3) & ~3;                  // rows of 16-byte groups
    float* ks = sh;                                   // [GC][dimP], already times w(cnt-1, s)
    float* vs = ks + GC * dimP;                       // [GC][GV]
    float* as = vs + GC * GV;                         // a_s
    float* ws = as + GC;                              // b_s, then w(cnt-1, s); ws[GC] = the chunk's whole decay
    pdl_trigger();
    const int c = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * GV;
    const int hq = h / (heads / qk_heads);
    const int b = table[B + 1 + 2 * c], q0 = table[B + 2 + 2 * c];
    const int row0 = cu_q[b] + q0, cnt = min(GC, cu_q[b + 1] - row0);
    pdl_wait();
    if (threadIdx.x < cnt) {
        const float2 g = *reinterpret_cast<const float2*>(&ab[((size_t)(row0 + threadIdx.x) * heads + h) * 2]);
        as[threadIdx.x] = g.x;
        ws[threadIdx.x] = g.y;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float p = 1.f;
        for (int s = cnt - 1; s >= 0; --s) { ws[s] *= p; p *= as[s]; }
        ws[GC] = p;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < cnt * dimP; idx += 256) {
        const int s = idx / dimP, i = idx - s * dimP;
        ks[idx] = i < dim ? k[(size_t)(row0 + s) * qk_stride + hq * dim + i] * ws[s] : 0.f;
    }
    for (int idx = threadIdx.x; idx < cnt * GV; idx += 256) {
        const int s = idx / GV, j = idx - s * GV;
        vs[idx] = (j0 + j < vdim) ? Cvt<T>::to_f32(v[(size_t)(row0 + s) * v_stride + h * vdim + j0 + j]) : 0.f;
    }
    __syncthreads();
    if (blockIdx.z == 0) {
        if (threadIdx.x == 0) CD[(size_t)c * heads + h] = ws[GC];
        if (NL != nullptr)
            for (int i = threadIdx.x; i < dim; i += 256) {
                float n = 0.f;
                for (int s = 0; s < cnt; ++s) n += ks[s * dimP + i];
                NL[((size_t)c * heads + h) * dim + i] = n;
            }
    }
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int groups = (dim + 63) / 64;               // 16-byte groups of rows per thread
    const int i0 = ty * 4 * groups;
    float acc[16][4];
#pragma unroll
    for (int r = 0; r < 16; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
    for (int s = 0; s < cnt; ++s) {
        const float4 vv = *reinterpret_cast<const float4*>(&vs[s * GV + 4 * tx]);
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

// grid (sequence, head, blocks over dim * vdim (+ dim with a normaliser)); a thread owns one element of the state (or of
// the normaliser) through all chunks
__global__ void __launch_bounds__(256)
gated_chunk_carry_kernel(float* __restrict__ LS, float* __restrict__ NL, const float* __restrict__ CD, float* __restrict__ state,
                         float* __restrict__ nstate, const int* __restrict__ table, const int* __restrict__ cu_q,
                         const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int ne = dim * vdim;
    if (e >= ne + (nstate != nullptr ? dim : 0)) return;
    const int c0 = table[b], c1 = table[b + 1];
    const bool of_n = e >= ne;
    float* S = of_n ? nstate + ((size_t)seq_slot[b] * heads + h) * dim + (e - ne)
                    : state + ((size_t)seq_slot[b] * heads + h) * ne + e;
    const size_t step = (size_t)heads * (of_n ? dim : ne);
    float* p = of_n ? NL + ((size_t)c0 * heads + h) * dim + (e - ne) : LS + ((size_t)c0 * heads + h) * ne + e;
    const float* cd = CD + (size_t)c0 * heads + h;
    pdl_wait();
    float s = *S;
    for (int c = c0; c < c1; c += 8) {                   // eight chunks' sums on their way at once; the chain is the FMAs alone
        float l[8], d[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            l[u] = (c + u < c1) ? p[(size_t)u * step] : 0.f;
            d[u] = (c + u < c1) ? cd[(size_t)u * heads] : 1.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (c + u < c1) {
                p[(size_t)u * step] = s;                 // the state before chunk c + u
                s = fmaf(d[u], s, l[u]);
            }
        p += 8 * step;
        cd += 8 * (size_t)heads;
    }
    *S = s;
}

// grid (chunk, head, ceil(vdim / GV)); 256 threads as a 16 x 16 grid of 4 x 4 tiles
template <typename T>
__global__ void __launch_bounds__(256)
gated_chunk_out_kernel(const float* __restrict__ q, const float* __restrict__ k, int qk_heads, int qk_stride,
                       const float* __restrict__ ab, const T* __restrict__ v, int v_stride, const float* __restrict__ LS,
                       const float* __restrict__ NL, float* __restrict__ o, float* __restrict__ qn,
                       const int* __restrict__ table, const int* __restrict__ cu_q, int B, int heads, int dim, int vdim) {
    extern __shared__ __align__(16) float sh[];
    float* qt = sh;                                   // [dim][GC_LD]: q transposed
    float* kt = qt + dim * GC_LD;                     // [dim][GC_LD]: k transposed; later the state S0 as [dim][GV]
    float* vs = kt + dim * GC_LD;                     // [GC][GV]
    float* at = vs + GC * GV;                         // [GC (s)][GC_LD (t)]: w(t, s), then the weighted scores, transposed
    float* as = at + GC * GC_LD;                      // a_t
    float* bs = as + GC;                              // b_s
    float* pt = bs + GC;                              // P_t
    pdl_trigger();
    const int c = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * GV;
    const int hq = h / (heads / qk_heads);
    const int b = table[B + 1 + 2 * c], q0 = table[B + 2 + 2 * c];
    const int row0 = cu_q[b] + q0, cnt = min(GC, cu_q[b + 1] - row0);
    pdl_wait();
    if (threadIdx.x < GC) {
        float2 g = make_float2(1.f, 0.f);
        if (threadIdx.x < cnt) g = *reinterpret_cast<const float2*>(&ab[((size_t)(row0 + threadIdx.x) * heads + h) * 2]);
        as[threadIdx.x] = g.x;
        bs[threadIdx.x] = g.y;
    }
    for (int idx = threadIdx.x; idx < GC * dim; idx += 256) {
        const int s = idx / dim, i = idx - s * dim;
        const bool in = s < cnt;
        qt[i * GC_LD + s] = in ? q[(size_t)(row0 + s) * qk_stride + hq * dim + i] : 0.f;
        kt[i * GC_LD + s] = in ? k[(size_t)(row0 + s) * qk_stride + hq * dim + i] : 0.f;
    }
    for (int idx = threadIdx.x; idx < GC * GV; idx += 256) {
        const int s = idx / GV, j = idx - s * GV;
        vs[idx] = (s < cnt && j0 + j < vdim) ? Cvt<T>::to_f32(v[(size_t)(row0 + s) * v_stride + h * vdim + j0 + j]) : 0.f;
    }
    __syncthreads();
    // the running products: thread s multiplies b_s on by a_(s+1), a_(s+2), ...; one more thread forms P_t
    if (threadIdx.x < GC) {
        const int s = threadIdx.x;
        float run = bs[s];
        at[s * GC_LD + s] = run;
        for (int t = s + 1; t < GC; ++t) { run *= as[t]; at[s * GC_LD + t] = run; }
    } else if (threadIdx.x == GC) {
        float p = 1.f;
        for (int t = 0; t < GC; ++t) { p *= as[t]; pt[t] = p; }
    }
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;        // rows (t) 4 ty .., columns 4 tx ..
    float a[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x) { a[x][0] = a[x][1] = a[x][2] = a[x][3] = 0.f; }
    if (tx <= ty) {                                      // tiles above the diagonal are zero
        for (int i = 0; i < dim; ++i) {
            const float4 qq = *reinterpret_cast<const float4*>(&qt[i * GC_LD + 4 * ty]);
            const float4 kk = *reinterpret_cast<const float4*>(&kt[i * GC_LD + 4 * tx]);
            const float qv[4] = {qq.x, qq.y, qq.z, qq.w}, kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) a[x][y] = fmaf(qv[x], kv[y], a[x][y]);
        }
    }
    __syncthreads();                                     // the products are in place; k is used up
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int t = 4 * ty + x, s = 4 * tx + y;
            at[s * GC_LD + t] = (s <= t) ? a[x][y] * at[s * GC_LD + t] : 0.f;
        }
    const float* S0 = LS + (((size_t)c * heads + h) * dim) * vdim;
    for (int idx = threadIdx.x; idx < dim * GV; idx += 256) {
        const int i = idx / GV, j = idx - i * GV;
        kt[idx] = (j0 + j < vdim) ? S0[(size_t)i * vdim + j0 + j] : 0.f;
    }
    __syncthreads();
    if (qn != nullptr && blockIdx.z == 0 && threadIdx.x < cnt) {
        const int t = threadIdx.x;
        const float* n0 = NL + ((size_t)c * heads + h) * dim;
        float inside = 0.f, before = 0.f;
        for (int s = 0; s <= t; ++s) inside += at[s * GC_LD + t];
        for (int i = 0; i < dim; ++i) before = fmaf(qt[i * GC_LD + t], n0[i], before);
        qn[(size_t)(row0 + t) * heads + h] = fmaf(pt[t], before, inside);
    }
    float o1[4][4], o2[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) { o1[x][y] = 0.f; o2[x][y] = 0.f; }
    const int s_end = min(cnt, 4 * ty + 4);              // later keys have zero scores for these rows
    for (int s = 0; s < s_end; ++s) {
        const float4 aa = *reinterpret_cast<const float4*>(&at[s * GC_LD + 4 * ty]);
        const float4 vv = *reinterpret_cast<const float4*>(&vs[s * GV + 4 * tx]);
        const float av[4] = {aa.x, aa.y, aa.z, aa.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) o1[x][y] = fmaf(av[x], vw[y], o1[x][y]);
    }
    for (int i = 0; i < dim; ++i) {
        const float4 qq = *reinterpret_cast<const float4*>(&qt[i * GC_LD + 4 * ty]);
        const float4 ss = *reinterpret_cast<const float4*>(&kt[i * GV + 4 * tx]);
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
                if (j < vdim) o[(size_t)(row0 + t) * heads * vdim + h * vdim + j] = fmaf(pt[t], o2[x][y], o1[x][y]);
            }
    }
}

template <typename T>
static int launch_gated_chunked(const float* q, const float* k, int qk_heads, int qk_stride, const float* ab, const void* v,
                                int v_stride, float* state, float* nstate, float* o, float* qn, float* scratch,
                                const int* table, int n_chunks, const int* cu_q, const int* seq_slot, int B, int heads,
                                int dim, int vdim, cudaStream_t st) {
    if (B <= 0 || n_chunks <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || heads <= 0 || heads > 65535 || B > 65535 || qk_heads <= 0 || heads % qk_heads)
        return RF_ERR_UNSUPPORTED;
    if ((nstate == nullptr) != (qn == nullptr)) return RF_ERR_BAD_ARG;
    float* LS = scratch;                                           // [n_chunks, heads, dim, vdim]
    float* CD = LS + (size_t)n_chunks * heads * dim * vdim;        // [n_chunks, heads]
    float* NL = nstate != nullptr ? CD + (size_t)n_chunks * heads : nullptr;   // [n_chunks, heads, dim]
    const int vz = (vdim + GV - 1) / GV;
    const size_t smem1 = (size_t)(GC * ((dim + 3) & ~3) + GC * GV + 2 * GC + 4) * sizeof(float);
    const size_t smem3 = (size_t)(2 * dim * GC_LD + GC * GV + GC * GC_LD + 3 * GC) * sizeof(float);
    static size_t set1 = 48 * 1024, set3 = 48 * 1024;
    if (smem1 > set1) {
        cudaError_t e = cudaFuncSetAttribute(gated_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (e != cudaSuccess) return (int)e;
        set1 = smem1;
    }
    if (smem3 > set3) {
        cudaError_t e = cudaFuncSetAttribute(gated_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
        if (e != cudaSuccess) return (int)e;
        set3 = smem3;
    }
    rf_launch(gated_chunk_state_kernel<T>, dim3(n_chunks, heads, vz), dim3(256), smem1, st, k, qk_heads, qk_stride, ab,
              reinterpret_cast<const T*>(v), v_stride, LS, NL, CD, table, cu_q, B, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    const int elements = dim * vdim + (nstate != nullptr ? dim : 0);
    rf_launch(gated_chunk_carry_kernel, dim3(B, heads, (elements + 255) / 256), dim3(256), 0, st, LS, NL, (const float*)CD, state,
              nstate, table, cu_q, seq_slot, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    rf_launch(gated_chunk_out_kernel<T>, dim3(n_chunks, heads, vz), dim3(256), smem3, st, q, k, qk_heads, qk_stride, ab,
              reinterpret_cast<const T*>(v), v_stride, (const float*)LS, (const float*)NL, o, qn, table, cu_q, B, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    return 0;
}

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
// The scalar recurrence of a prompt step in chunks of 64 tokens (see above).  scratch: float, n_chunks * heads *
// (dim * vdim + 1 (+ dim with a normaliser)); table: first[B+1], then n_chunks pairs (sequence, first row of the chunk among
// the sequence's new tokens).  The other arguments are rf_gated_scan's.
int rf_gated_chunked(int dtype, const float* q, const float* k, int qk_heads, int qk_stride, const float* ab, const void* v,
                     int v_stride, float* state, float* nstate, float* o, float* qn, float* scratch, const int* table,
                     int n_chunks, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    return dtype == 0 ? launch_gated_chunked<float>(q, k, qk_heads, qk_stride, ab, v, v_stride, state, nstate, o, qn, scratch, table,
                                                    n_chunks, cu_q, seq_slot, B, heads, dim, vdim, st)
                      : launch_gated_chunked<__nv_bfloat16>(q, k, qk_heads, qk_stride, ab, v, v_stride, state, nstate, o, qn, scratch,
                                                            table, n_chunks, cu_q, seq_slot, B, heads, dim, vdim, st);
}
}
