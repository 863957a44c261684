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
//                  independent of each other, so blocks never talk.  A lane owns a column, each of the four warps a
//                  slice of ROWS rows, kept in registers over the step's tokens.  Per token the warps' partial r_k and
//                  r_q meet in shared memory (two buffers in turn: one barrier a token) and are added in warp order.
//                  The order of every sum is fixed by (dim, position) alone: how a prompt is cut into steps and what
//                  else is in the batch change no bit.
#include "common.cuh"

#define DL_WARPS 4
#define DL_COLS 32

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
    for (int g = warp; g < G; g += nwarp) {                 // a warp per q/k head
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
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
        const int h = i / D;
        const float x = a[(size_t)t * H * D + i] + load_vec(dt_bias, vec_is_f32, i);
        const float sp = fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
        decay[(size_t)t * H * D + i] = expf(-expf(load_vec(a_log, vec_is_f32, h)) * sp);
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        beta[(size_t)t * H + h] = 1.f / (1.f + expf(-Cvt<T>::to_f32(beta_src[(size_t)t * beta_stride + h])));
}

// grid (ceil(vdim / 32), heads, sequences); 128 threads.  DP = DL_WARPS * ROWS >= dim; rows beyond dim hold zeros.
template <int ROWS>
__global__ void __launch_bounds__(DL_WARPS * 32)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ kq,
                  const float* __restrict__ decay, const float* __restrict__ beta, const float* __restrict__ v, int v_stride,
                  float* __restrict__ state, float* __restrict__ o, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_slot, int H, int G, int D, int V) {
    constexpr int DP = DL_WARPS * ROWS;
    constexpr int DL_TOK = ROWS > 32 ? 8 : 16;      // tokens staged in shared memory at a time
    __shared__ __align__(16) float sk[DL_TOK][DP], sq[DL_TOK][DP], sg[DL_TOK][DP];
    __shared__ float sv[DL_TOK][DL_COLS], sb[DL_TOK], skq[DL_TOK];
    __shared__ float red[2][DL_WARPS][2][DL_COLS];
    pdl_trigger();
    const int b = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * DL_COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hg = h / (H / G);
    const int t0 = cu_q[b], n = cu_q[b + 1] - t0;
    const int col = j0 + lane;
    const bool live = col < V;
    float* S = state + ((size_t)seq_slot[b] * H + h) * D * V;
    pdl_wait();
    float s[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = warp * ROWS + r;
        s[r] = (live && i < D) ? S[(size_t)i * V + col] : 0.f;
    }
    for (int base = 0; base < n; base += DL_TOK) {
        const int cnt = min(DL_TOK, n - base);
        __syncthreads();                                    // the stage before is used up
        for (int i = tid; i < cnt * DP; i += DL_WARPS * 32) {
            const int tt = i / DP, d = i - tt * DP;
            const size_t t = (size_t)(t0 + base + tt);
            const bool in = d < D;
            sk[tt][d] = in ? kn[(t * G + hg) * D + d] : 0.f;
            sq[tt][d] = in ? qn[(t * G + hg) * D + d] : 0.f;
            sg[tt][d] = in ? decay[(t * H + h) * D + d] : 1.f;
        }
        for (int i = tid; i < cnt * DL_COLS; i += DL_WARPS * 32) {
            const int tt = i / DL_COLS, c = i - tt * DL_COLS;
            sv[tt][c] = j0 + c < V ? v[(size_t)(t0 + base + tt) * v_stride + h * V + j0 + c] : 0.f;
        }
        if (tid < cnt) {
            sb[tid] = beta[(size_t)(t0 + base + tid) * H + h];
            skq[tid] = kq[(size_t)(t0 + base + tid) * G + hg];
        }
        __syncthreads();
        for (int tt = 0; tt < cnt; ++tt) {
            const float* kk = &sk[tt][warp * ROWS];
            const float* qq = &sq[tt][warp * ROWS];
            const float* gg = &sg[tt][warp * ROWS];
            float pk[4] = {0.f, 0.f, 0.f, 0.f}, pq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 g4 = *reinterpret_cast<const float4*>(gg + r);
                const float4 k4 = *reinterpret_cast<const float4*>(kk + r);
                const float4 q4 = *reinterpret_cast<const float4*>(qq + r);
                s[r + 0] *= g4.x; pk[0] = fmaf(s[r + 0], k4.x, pk[0]); pq[0] = fmaf(s[r + 0], q4.x, pq[0]);
                s[r + 1] *= g4.y; pk[1] = fmaf(s[r + 1], k4.y, pk[1]); pq[1] = fmaf(s[r + 1], q4.y, pq[1]);
                s[r + 2] *= g4.z; pk[2] = fmaf(s[r + 2], k4.z, pk[2]); pq[2] = fmaf(s[r + 2], q4.z, pq[2]);
                s[r + 3] *= g4.w; pk[3] = fmaf(s[r + 3], k4.w, pk[3]); pq[3] = fmaf(s[r + 3], q4.w, pq[3]);
            }
            const int par = tt & 1;
            red[par][warp][0][lane] = (pk[0] + pk[1]) + (pk[2] + pk[3]);
            red[par][warp][1][lane] = (pq[0] + pq[1]) + (pq[2] + pq[3]);
            __syncthreads();
            float rk = red[par][0][0][lane], rq = red[par][0][1][lane];
#pragma unroll
            for (int w = 1; w < DL_WARPS; ++w) { rk += red[par][w][0][lane]; rq += red[par][w][1][lane]; }
            const float u = sb[tt] * (sv[tt][lane] - rk);
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kk + r);
                s[r + 0] = fmaf(k4.x, u, s[r + 0]);
                s[r + 1] = fmaf(k4.y, u, s[r + 1]);
                s[r + 2] = fmaf(k4.z, u, s[r + 2]);
                s[r + 3] = fmaf(k4.w, u, s[r + 3]);
            }
            if (warp == 0 && live) o[(size_t)(t0 + base + tt) * H * V + h * V + col] = fmaf(skq[tt], u, rq);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int i = warp * ROWS + r;
        if (live && i < D) S[(size_t)i * V + col] = s[r];
    }
}

template <int ROWS>
static int launch_scan(const float* qn, const float* kn, const float* kq, const float* decay, const float* beta, const float* v,
                       int v_stride, float* state, float* o, const int* cu_q, const int* seq_slot, int B, int H, int G, int D,
                       int V, cudaStream_t st) {
    rf_launch(delta_scan_kernel<ROWS>, dim3((V + DL_COLS - 1) / DL_COLS, H, B), dim3(DL_WARPS * 32), 0, st, qn, kn, kq, decay,
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
    if (dtype == 0)
        rf_launch(delta_prepare_kernel<float>, dim3(T_), dim3(128), 0, st, qkv, qkv_stride, a, dt_bias, a_log, vec_is_f32,
                  reinterpret_cast<const float*>(beta_src), beta_stride, qn, kn, kq, decay, beta, H, G, D, q_scale, unit_eps);
    else
        rf_launch(delta_prepare_kernel<__nv_bfloat16>, dim3(T_), dim3(128), 0, st, qkv, qkv_stride, a, dt_bias, a_log, vec_is_f32,
                  reinterpret_cast<const __nv_bfloat16*>(beta_src), beta_stride, qn, kn, kq, decay, beta, H, G, D, q_scale, unit_eps);
    RF_LAUNCH_CHECK();
    return 0;
}
// state float [slots, H, D, V]; v float [T, v_stride] with head h's values at columns h*V..; o float [T, H*V]; cu_q [B+1]
int rf_delta_scan(const float* qn, const float* kn, const float* kq, const float* decay, const float* beta, const float* v,
                  int v_stride, float* state, float* o, const int* cu_q, const int* seq_slot, int B, int H, int G, int D, int V,
                  cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || H > 65535 || B > 65535) return RF_ERR_BAD_ARG;
    if (D <= 32) return launch_scan<8>(qn, kn, kq, decay, beta, v, v_stride, state, o, cu_q, seq_slot, B, H, G, D, V, st);
    if (D <= 64) return launch_scan<16>(qn, kn, kq, decay, beta, v, v_stride, state, o, cu_q, seq_slot, B, H, G, D, V, st);
    if (D <= 128) return launch_scan<32>(qn, kn, kq, decay, beta, v, v_stride, state, o, cu_q, seq_slot, B, H, G, D, V, st);
    if (D <= 256) return launch_scan<64>(qn, kn, kq, decay, beta, v, v_stride, state, o, cu_q, seq_slot, B, H, G, D, V, st);
    return RF_ERR_UNSUPPORTED;
}
}
