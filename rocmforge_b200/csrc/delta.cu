// The gated delta rule: a matrix state per head that decays per key channel and is corrected, not just added to:
//   S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t      (S is [dim, vdim])
// so the read-out sees the token's own write.  With S' = diag(g_t) S both products that a token needs are taken from S'
// in one pass over the state, r_k = S'^T k_t and r_q = S'^T q_t, because o_t = r_q + (k_t . q_t) u_t; the state is read
// once and written once per token.  Everything here is 32-bit.
//
//   delta_prepare  q and k heads made unit vectors (x / sqrt(sum x^2 + unit_eps), q also times q_scale), their dot
//                  products k . q, beta = sigmoid of the projection's columns, and the decays
//                  g = exp(-exp(A_log_h) softplus(a + dt_bias)) per head and key channel
//   delta_scan     the recurrence, token by token.  A block owns (sequence, head, 32 value columns): the columns of S are
//                  independent of each other, so blocks never talk.  Four lanes share a column, each with a quarter of
//                  its rows in registers over the step's tokens; per token their partial r_k and r_q meet by shuffles.
//                  The order of every sum is fixed by (dim, position) alone: how a prompt is cut into steps and what
//                  else is in the batch change no bit.
#include "common.cuh"

#define DL_WARPS 4

template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ qkv, int qkv_stride, const float* __restrict__ a, const void* __restrict__ dt_bias,
                     const void* __restrict__ a_log, int vec_is_f32, const T* __restrict__ beta_src, int beta_stride,
                     float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ kq, float* __restrict__ decay,
                     float* __restrict__ beta, int H, int G, int D, float q_scale, float unit_eps) {
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    pdl_wait();
    const float* row = qkv + (size_t)t * qkv_stride;
    // few tokens: a token's heads and channels are spread over gridDim.y blocks
    for (int g = blockIdx.y * nwarp + warp; g < G; g += gridDim.y * nwarp) {                 // a warp per q/k head
        const float* q = row + g * D;
        const float* k = row + (G + g) * D;
        float sq = 0.f, sk = 0.f, dot = 0.f;
        for (int e = lane; e < D; e += 32) { const float x = q[e], y = k[e]; sq += x * x; sk += y * y; dot += x * y; }
        sq = warp_sum(sq); sk = warp_sum(sk); dot = warp_sum(dot);
        const float rq = q_scale / sqrtf(sq + unit_eps), rk = 1.f / sqrtf(sk + unit_eps);
        for (int e = lane; e < D; e += 32) {
            qn[((size_t)t * G + g) * D + e] = q[e] * rq;
            kn[((size_t)t * G + g) * D + e] = k[e] * rk;
        }
        if (lane == 0) kq[(size_t)t * G + g] = dot * rq * rk;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H * D; i += gridDim.y * blockDim.x) {
        const int h = i / D;
        const float x = a[(size_t)t * H * D + i] + load_vec(dt_bias, vec_is_f32, i);
        const float sp = fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
        decay[(size_t)t * H * D + i] = expf(-expf(load_vec(a_log, vec_is_f32, h)) * sp);
    }
    for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < H; h += gridDim.y * blockDim.x)
        beta[(size_t)t * H + h] = 1.f / (1.f + expf(-Cvt<T>::to_f32(beta_src[(size_t)t * beta_stride + h])));
}

// grid (ceil(vdim / COLS), heads, sequences); 128 threads.  LPC lanes share a value column (a warp owns 32 / LPC columns, a
// block COLS = 128 / LPC); DP = LPC * ROWS >= dim, a multiple of 4 LPC; rows beyond dim hold zeros.  Of every 4 LPC rows of
// the state the lane with number rg inside its column holds rows 4 rg .. 4 rg + 3, so that the lanes' 16-byte reads of q, k
// and the decays from shared memory lie in a row.  A column's partial products meet by log2(LPC) shuffles; the warps of a block never wait for each other
// inside a stage.  The tokens' q, k, decays, values, beta and k . q are copied asynchronously, a stage of TOK tokens
// ahead of the arithmetic.
__device__ __forceinline__ void dl_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dl_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int ROWS, int LPC>
__global__ void __launch_bounds__(DL_WARPS * 32)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ kq,
                  const float* __restrict__ decay, const float* __restrict__ beta, const float* __restrict__ v, int v_stride,
                  float* __restrict__ state, float* __restrict__ o, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_slot, int H, int G, int D, int V) {
    constexpr int DP = LPC * ROWS;                                   // rows of the padded state
    constexpr int COLS = DL_WARPS * 32 / LPC;                        // value columns of a block
    constexpr int TOK = DP <= 64 ? 16 : (DP <= 128 ? 8 : 4);         // tokens of a stage
    constexpr int NT = DL_WARPS * 32;
    __shared__ __align__(16) float sk[2][TOK][DP], sq[2][TOK][DP], sg[2][TOK][DP];
    __shared__ __align__(16) float sv[2][TOK][COLS];
    __shared__ float sb[2][TOK], skq[2][TOK];
    pdl_trigger();
    const int b = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rg = lane % LPC, cl = warp * (32 / LPC) + lane / LPC;            // this lane's rows inside every 16, its column in the block
    const int hg = h / (H / G);
    const int t0 = cu_q[b], n = cu_q[b + 1] - t0;
    const int col = j0 + cl;
    const bool live = col < V;
    float* S = state + ((size_t)seq_slot[b] * H + h) * D * V;
    // what no copy ever writes: rows beyond dim (k = q = 0, decay 1) and columns beyond vdim (value 0)
    for (int i = tid; i < 2 * TOK * DP; i += NT) {
        const int d = i % DP;
        if (d >= D) { (&sk[0][0][0])[i] = 0.f; (&sq[0][0][0])[i] = 0.f; (&sg[0][0][0])[i] = 1.f; }
    }
    for (int i = tid; i < 2 * TOK * COLS; i += NT)
        if (j0 + i % COLS >= V) (&sv[0][0][0])[i] = 0.f;
    const bool vec = (D & 3) == 0;
    pdl_wait();
    auto stage_in = [&](int base, int buf) {
        const int cnt = min(TOK, n - base);
        if (vec) {
            const int dq = D >> 2;
            for (int i = tid; i < cnt * dq; i += NT) {
                const int tt = i / dq, d = (i - tt * dq) * 4;
                const size_t t = (size_t)(t0 + base + tt);
                dl_copy16(&sk[buf][tt][d], kn + (t * G + hg) * D + d);
                dl_copy16(&sq[buf][tt][d], qn + (t * G + hg) * D + d);
                dl_copy16(&sg[buf][tt][d], decay + (t * H + h) * D + d);
            }
        } else {
            for (int i = tid; i < cnt * D; i += NT) {
                const int tt = i / D, d = i - tt * D;
                const size_t t = (size_t)(t0 + base + tt);
                dl_copy4(&sk[buf][tt][d], kn + (t * G + hg) * D + d);
                dl_copy4(&sq[buf][tt][d], qn + (t * G + hg) * D + d);
                dl_copy4(&sg[buf][tt][d], decay + (t * H + h) * D + d);
            }
        }
        const int nc = min(COLS, V - j0);
        for (int i = tid; i < cnt * nc; i += NT) {
            const int tt = i / nc, c = i - tt * nc;
            dl_copy4(&sv[buf][tt][c], v + (size_t)(t0 + base + tt) * v_stride + h * V + j0 + c);
        }
        if (tid < cnt) {
            dl_copy4(&sb[buf][tid], beta + (size_t)(t0 + base + tid) * H + h);
            dl_copy4(&skq[buf][tid], kq + (size_t)(t0 + base + tid) * G + hg);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float s[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = (r >> 2) * (4 * LPC) + rg * 4 + (r & 3);
        s[r] = (live && i < D) ? S[(size_t)i * V + col] : 0.f;
    }
    if (n > 0) stage_in(0, 0);
    for (int base = 0, buf = 0; base < n; base += TOK, buf ^= 1) {
        const int cnt = min(TOK, n - base);
        if (base + TOK < n) {
            stage_in(base + TOK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                    // this stage's copies of every thread have landed
        float4 g4[ROWS / 4], k4[ROWS / 4], q4[ROWS / 4];
        auto fetch = [&](int tt) {
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                g4[r] = *reinterpret_cast<const float4*>(&sg[buf][tt][rg * 4 + r * 4 * LPC]);
                k4[r] = *reinterpret_cast<const float4*>(&sk[buf][tt][rg * 4 + r * 4 * LPC]);
                q4[r] = *reinterpret_cast<const float4*>(&sq[buf][tt][rg * 4 + r * 4 * LPC]);
            }
        };
        for (int tt = 0; tt < cnt; ++tt) {
            fetch(tt);
            float pk[4] = {0.f, 0.f, 0.f, 0.f}, pq[4] = {0.f, 0.f, 0.f, 0.f};
            float4 kc[ROWS / 4];
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                kc[r] = k4[r];
                s[4 * r + 0] *= g4[r].x; pk[0] = fmaf(s[4 * r + 0], k4[r].x, pk[0]); pq[0] = fmaf(s[4 * r + 0], q4[r].x, pq[0]);
                s[4 * r + 1] *= g4[r].y; pk[1] = fmaf(s[4 * r + 1], k4[r].y, pk[1]); pq[1] = fmaf(s[4 * r + 1], q4[r].y, pq[1]);
                s[4 * r + 2] *= g4[r].z; pk[2] = fmaf(s[4 * r + 2], k4[r].z, pk[2]); pq[2] = fmaf(s[4 * r + 2], q4[r].z, pq[2]);
                s[4 * r + 3] *= g4[r].w; pk[3] = fmaf(s[4 * r + 3], k4[r].w, pk[3]); pq[3] = fmaf(s[4 * r + 3], q4[r].w, pq[3]);
            }
            float rk = (pk[0] + pk[1]) + (pk[2] + pk[3]), rq = (pq[0] + pq[1]) + (pq[2] + pq[3]);
            const float bt = sb[buf][tt], vt = sv[buf][tt][cl], kqt = skq[buf][tt];
#pragma unroll
            for (int m = 1; m < LPC; m <<= 1) { rk += __shfl_xor_sync(0xffffffffu, rk, m); rq += __shfl_xor_sync(0xffffffffu, rq, m); }
            const float u = bt * (vt - rk);
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                s[4 * r + 0] = fmaf(kc[r].x, u, s[4 * r + 0]);
                s[4 * r + 1] = fmaf(kc[r].y, u, s[4 * r + 1]);
                s[4 * r + 2] = fmaf(kc[r].z, u, s[4 * r + 2]);
                s[4 * r + 3] = fmaf(kc[r].w, u, s[4 * r + 3]);
            }
            if (rg == 0 && live) o[(size_t)(t0 + base + tt) * H * V + h * V + col] = fmaf(kqt, u, rq);
        }
        __syncthreads();                                    // the stage is used up: the stage after next may land in it
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = (r >> 2) * (4 * LPC) + rg * 4 + (r & 3);
        if (live && i < D) S[(size_t)i * V + col] = s[r];
    }
}

template <int ROWS, int LPC>
static int launch_scan(const float* qn, const float* kn, const float* kq, const float* decay, const float* beta, const float* v,
                       int v_stride, float* state, float* o, const int* cu_q, const int* seq_slot, int B, int H, int G, int D,
                       int V, cudaStream_t st) {
    constexpr int COLS = DL_WARPS * 32 / LPC;
    rf_launch(delta_scan_kernel<ROWS, LPC>, dim3((V + COLS - 1) / COLS, H, B), dim3(DL_WARPS * 32), 0, st, qn, kn, kq, decay,
              beta, v, v_stride, state, o, cu_q, seq_slot, H, G, D, V);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {
// qkv float [T, qkv_stride]: q heads (G x D), k heads (G x D), then values; a float [T, H*D]; dt_bias [H*D] and a_log [H] of one
// dtype (vec_is_f32); beta_src [T, beta_stride] of dtype, H columns.  Out: qn, kn float [T, G*D], kq float [T, G], decay float
// [T, H*D], beta float [T, H].
int rf_delta_prepare(int dtype, const float* qkv, int qkv_stride, const float* a, const void* dt_bias, const void* a_log,
                     int vec_is_f32, const void* beta_src, int beta_stride, float* qn, float* kn, float* kq, float* decay,
                     float* beta, int H, int G, int D, float q_scale, float unit_eps, int T_, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0) return RF_ERR_BAD_ARG;
    int by = T_ >= 512 ? 1 : (H * D + 511) / 512;           // about four decays a thread when there are few tokens
    if (by > 32) by = 32;
    if (dtype == 0)
        rf_launch(delta_prepare_kernel<float>, dim3(T_, by), dim3(128), 0, st, qkv, qkv_stride, a, dt_bias, a_log, vec_is_f32,
                  reinterpret_cast<const float*>(beta_src), beta_stride, qn, kn, kq, decay, beta, H, G, D, q_scale, unit_eps);
    else
        rf_launch(delta_prepare_kernel<__nv_bfloat16>, dim3(T_, by), dim3(128), 0, st, qkv, qkv_stride, a, dt_bias, a_log, vec_is_f32,
                  reinterpret_cast<const __nv_bfloat16*>(beta_src), beta_stride, qn, kn, kq, decay, beta, H, G, D, q_scale, unit_eps);
    RF_LAUNCH_CHECK();
    return 0;
}
// state float [slots, H, D, V]; v float [T, v_stride] with head h's values at columns h*V..; o float [T, H*V]; cu_q [B+1]
int rf_delta_scan(const float* qn, const float* kn, const float* kq, const float* decay, const float* beta, const float* v,
                  int v_stride, float* state, float* o, const int* cu_q, const int* seq_slot, int B, int H, int G, int D, int V,
                  int one_token, int lanes, cudaStream_t st) {
    if (B <= 0) return 0;
    if (lanes != 0 && lanes != 4 && lanes != 8) return RF_ERR_BAD_ARG;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || H > 65535 || B > 65535) return RF_ERR_BAD_ARG;
#define DL_GO(ROWS, LPC) return launch_scan<ROWS, LPC>(qn, kn, kq, decay, beta, v, v_stride, state, o, cu_q, seq_slot, B, H, G, D, V, st)
    // Steps of one token a sequence (the state is read and written once, nothing else): four lanes a column.  Steps with
    // longer portions: eight lanes a column (twice the blocks, half the chain of each; fetching the next token's operands
    // into registers ahead of the chain was measured and cost more in registers than it hid).  The two forms add a column's products in another order: a difference of rounding between a token
    // decoded alone and the same token inside a portion, none between two cuts into portions.
    const int lpc = lanes > 0 ? lanes : (one_token ? 4 : 8);
    const int rows = (D + 4 * lpc - 1) / (4 * lpc) * 4;        // rows a lane, a multiple of 4
    if (lpc == 4) { if (rows <= 8) DL_GO(8, 4); if (rows <= 16) DL_GO(16, 4); if (rows <= 32) DL_GO(32, 4); if (rows <= 64) DL_GO(64, 4); }
    if (lpc == 8) { if (rows <= 4) DL_GO(4, 8); if (rows <= 8) DL_GO(8, 8); if (rows <= 16) DL_GO(16, 8); if (rows <= 32) DL_GO(32, 8); }
#undef DL_GO
    return RF_ERR_UNSUPPORTED;
}
}
