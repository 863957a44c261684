// The matrix memory of xLSTM (mLSTM): per head a state S [dim, vdim] and a normaliser n [dim] that are gated by an
// exponential input gate and a sigmoid forget gate, both kept in the logarithm, with a running maximum m that keeps the
// exponentials in range:
//   li_t = cap tanh(zi_t / cap),  lf_t = log sigmoid(cap tanh(zf_t / cap))      (cap <= 0: not capped)
//   m_t = max(lf_t + m_(t-1), li_t)                                              (m starts at 0)
//   a_t = exp(lf_t + m_(t-1) - m_t),  b_t = exp(li_t - m_t)
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,  n_t = a_t n_(t-1) + b_t k_t             (the scalar form of gla_scan, csrc/gla.cu)
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                      (retention_gate with a denominator)
// Everything here is 32-bit.
//
//   mlstm_prepare   q (times q_scale) and k of the projection's rows as float [2, T, heads*dim]
//   mlstm_gates     the gates' chain: a block per (sequence, head) works through the sequence's new tokens in stretches
//                   of ML_TOK: all threads form li and lf, one thread runs the chain of maxima (two operations a token),
//                   all threads form a and b.  Leaves (a_t, b_t) as float [T, heads, 2], m_t as float [T, heads], and the
//                   last m in the state [slots, heads].  The chain's order is the tokens' order alone: how a prompt is cut
//                   into steps changes no bit.
#include "common.cuh"

#define ML_TOK 1024

template <typename T>
__global__ void mlstm_prepare_kernel(const T* __restrict__ src, int row_stride, int q_col, int k_col, float* __restrict__ qk,
                                     int width, float q_scale, int T_) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)T_ * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width, c = idx - t * width;
        qk[idx] = Cvt<T>::to_f32(src[t * row_stride + q_col + c]) * q_scale;
        qk[n + idx] = Cvt<T>::to_f32(src[t * row_stride + k_col + c]);
    }
}

__device__ __forceinline__ float ml_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// z float [T, 2*heads]: the input gate's pre-activations (bias included), then the forget gate's
__global__ void __launch_bounds__(256)
mlstm_gates_kernel(const float* __restrict__ z, float* __restrict__ ab, float* __restrict__ mt, float* __restrict__ mstate,
                   const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, float cap) {
    __shared__ float li[ML_TOK], lf[ML_TOK], mm[ML_TOK + 1];
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y;
    const int row0 = cu_q[b], row1 = cu_q[b + 1];
    float* mslot = mstate + (size_t)seq_slot[b] * heads + h;
    pdl_wait();
    if (threadIdx.x == 0) mm[0] = *mslot;
    for (int t0 = row0; t0 < row1; t0 += ML_TOK) {
        const int cnt = min(ML_TOK, row1 - t0);
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            float zi = z[(size_t)(t0 + i) * 2 * heads + h], zf = z[(size_t)(t0 + i) * 2 * heads + heads + h];
            if (cap > 0.f) { zi = cap * tanhf(zi / cap); zf = cap * tanhf(zf / cap); }
            li[i] = zi;
            lf[i] = ml_log_sigmoid(zf);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = mm[0];
            int i = 0;
            // eight tokens' gates are fetched before their links of the chain, so that the chain waits for no load
            for (; i + 8 <= cnt; i += 8) {
                float f[8], g[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) { f[u] = lf[i + u]; g[u] = li[i + u]; }
#pragma unroll
                for (int u = 0; u < 8; ++u) { m = fmaxf(f[u] + m, g[u]); mm[i + u + 1] = m; }
            }
            for (; i < cnt; ++i) { m = fmaxf(lf[i] + m, li[i]); mm[i + 1] = m; }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            const size_t e = (size_t)(t0 + i) * heads + h;
            ab[2 * e] = expf(lf[i] + mm[i] - mm[i + 1]);
            ab[2 * e + 1] = expf(li[i] - mm[i + 1]);
            mt[e] = mm[i + 1];
        }
        __syncthreads();
        if (threadIdx.x == 0) mm[0] = mm[cnt];
    }
    __syncthreads();
    if (threadIdx.x == 0) *mslot = mm[0];
}

template <typename T>
static int launch_prepare(const void* src, int row_stride, int q_col, int k_col, float* qk, int width, float q_scale, int T_,
                          cudaStream_t st) {
    const size_t n = (size_t)T_ * width;
    if (n == 0) return 0;
    const size_t blocks = (n + 255) / 256;
    rf_launch(mlstm_prepare_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st,
              reinterpret_cast<const T*>(src), row_stride, q_col, k_col, qk, width, q_scale, T_);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {
// dtype: 0 = float32, 1 = bfloat16 (of the projection's output)
int rf_mlstm_prepare(int dtype, const void* src, int row_stride, int q_col, int k_col, float* qk, int width, float q_scale,
                     int T_, cudaStream_t st) {
    return dtype == 0 ? launch_prepare<float>(src, row_stride, q_col, k_col, qk, width, q_scale, T_, st)
                      : launch_prepare<__nv_bfloat16>(src, row_stride, q_col, k_col, qk, width, q_scale, T_, st);
}
// max_new: the most new tokens of a sequence in this step (sizes the blocks)
int rf_mlstm_gates(const float* z, float* ab, float* mt, float* mstate, const int* cu_q, const int* seq_slot, int B, int heads,
                   float cap, int max_new, cudaStream_t st) {
    if (B <= 0) return 0;
    if (heads <= 0 || heads > 65535) return RF_ERR_UNSUPPORTED;
    int threads = 32;
    while (threads < 256 && threads < max_new) threads <<= 1;
    rf_launch(mlstm_gates_kernel, dim3(B, heads), dim3(threads), 0, st, z, ab, mt, mstate, cu_q, seq_slot, heads, cap);
    RF_LAUNCH_CHECK();
    return 0;
}
}
