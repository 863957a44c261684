// The parts of a Mamba-2 mixer (state-space duality) around its recurrence, which is the scalar form of gla_scan
// (csrc/gla.cu): S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t, with B as k, C as q, x as v, one (B, C) per group
// of heads.
//
//   conv_silu          a causal convolution per channel over the last `taps` inputs, then silu; the inputs before a step's
//                      first token come from the per-sequence state [slots, taps-1, channels] (zeros at a sequence's
//                      start), so a prompt may be cut anywhere.  Output 32-bit [T, channels].
//   conv_state_update  the state after the step: the last taps-1 inputs of every sequence
//   mamba_gates        dt = softplus(z + dt_bias), a = exp(-exp(A_log) dt): float [T, heads, 2] = (a, dt)
//   mamba_finish       y + D x, times silu(gate), RMS norm over each of `parts` equal parts of a row, times a weight,
//                      into the compute dtype
#include "common.cuh"

#define MB_MAX_TAPS 16

template <typename T>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const T* __restrict__ src, int row_stride, int col0, const float* __restrict__ state,
                 const void* __restrict__ w, const void* __restrict__ bias, int w_is_f32, float* __restrict__ out,
                 const int* __restrict__ tok_seq, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int C,
                 int taps) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    const int r = t - cu_q[b];                       // the token's index among its sequence's new tokens
    const float* old = state + (size_t)seq_slot[b] * (taps - 1) * C;
    pdl_wait();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = load_vec(bias, w_is_f32, c);
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;            // the last column weighs the current token
            const float x = r - back >= 0 ? Cvt<T>::to_f32(src[(size_t)(t - back) * row_stride + col0 + c])
                                          : old[(size_t)(taps - 1 + r - back) * C + c];
            acc = fmaf(load_vec(w, w_is_f32, c * taps + j), x, acc);
        }
        out[(size_t)t * C + c] = acc / (1.f + expf(-acc));
    }
}

// The same for rows whose channels come in whole groups of four (C, col0 and row_stride multiples of 4): a thread owns
// four neighbouring channels with their TAPS x 4 weights in registers and walks CV_TOK tokens; the inputs are 8- or
// 16-byte loads, the result one 16-byte store.  The sum of a channel runs over the taps in the same order as above.
#define CV_TOK 4

template <typename T> struct Vec4 {};
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float* x) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* x) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
        x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
    }
};

template <typename T, int TAPS>
__global__ void __launch_bounds__(256)
conv_silu_vec_kernel(const T* __restrict__ src, int row_stride, int col0, const float* __restrict__ state,
                     const void* __restrict__ w, const void* __restrict__ bias, int w_is_f32, float* __restrict__ out,
                     const int* __restrict__ tok_seq, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int C,
                     int T_) {
    pdl_trigger();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    const int t0 = blockIdx.x * CV_TOK;
    if (c >= C) return;
    float wt[TAPS][4], bs[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        bs[u] = load_vec(bias, w_is_f32, c + u);
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wt[j][u] = load_vec(w, w_is_f32, (c + u) * TAPS + j);
    }
    pdl_wait();
    for (int t = t0; t < t0 + CV_TOK && t < T_; ++t) {
        const int b = tok_seq[t];
        const int r = t - cu_q[b];
        const float* old = state + (size_t)seq_slot[b] * (TAPS - 1) * C;
        float acc[4] = {bs[0], bs[1], bs[2], bs[3]};
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
            const int back = TAPS - 1 - j;
            float x[4];
            if (r - back >= 0) Vec4<T>::load(src + (size_t)(t - back) * row_stride + col0 + c, x);
            else Vec4<float>::load(old + (size_t)(TAPS - 1 + r - back) * C + c, x);
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = fmaf(wt[j][u], x[u], acc[u]);
        }
        float4 y;
        y.x = acc[0] / (1.f + expf(-acc[0])); y.y = acc[1] / (1.f + expf(-acc[1]));
        y.z = acc[2] / (1.f + expf(-acc[2])); y.w = acc[3] / (1.f + expf(-acc[3]));
        *reinterpret_cast<float4*>(out + (size_t)t * C + c) = y;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* __restrict__ src, int row_stride, int col0, float* __restrict__ state,
                         const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int C, int taps) {
    pdl_trigger();
    const int b = blockIdx.x;
    const int row0 = cu_q[b], n = cu_q[b + 1] - row0;
    float* st = state + (size_t)seq_slot[b] * (taps - 1) * C;
    pdl_wait();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float keep[MB_MAX_TAPS];
#pragma unroll
        for (int i = 0; i < MB_MAX_TAPS; ++i) {
            if (i < taps - 1) {
                const int r = n - (taps - 1) + i;     // index among the new tokens of the input that lands in entry i
                keep[i] = r >= 0 ? Cvt<T>::to_f32(src[(size_t)(row0 + r) * row_stride + col0 + c])
                                 : st[(size_t)(taps - 1 + r) * C + c];
            }
        }
#pragma unroll
        for (int i = 0; i < MB_MAX_TAPS; ++i)
            if (i < taps - 1) st[(size_t)i * C + c] = keep[i];
    }
}

__global__ void mamba_gates_kernel(const float* __restrict__ z, const void* __restrict__ dt_bias, const void* __restrict__ a_log,
                                   int v_is_f32, float* __restrict__ ab, int heads, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int h = (int)(idx % heads);
        const float x = z[idx] + load_vec(dt_bias, v_is_f32, h);
        const float dt = fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
        ab[2 * idx] = expf(-expf(load_vec(a_log, v_is_f32, h)) * dt);
        ab[2 * idx + 1] = dt;
    }
}

// A block per (token, part).  y float [T, inner]; x float rows of x_stride; gate rows of the compute dtype.
template <typename T>
__global__ void __launch_bounds__(256)
mamba_finish_kernel(const float* __restrict__ y, const float* __restrict__ x, int x_stride, const T* __restrict__ gate,
                    int gate_stride, const void* __restrict__ skip, const void* __restrict__ norm_w, int v_is_f32,
                    T* __restrict__ out, int inner, int parts, int vdim, float eps) {
    extern __shared__ float row[];                   // [inner / parts] + 34
    const int len = inner / parts;
    float* red = row + len;
    pdl_trigger();
    const int t = blockIdx.x, c0 = blockIdx.y * len;
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const int c = c0 + i;
        const float g = Cvt<T>::to_f32(gate[(size_t)t * gate_stride + c]);
        float v = y[(size_t)t * inner + c] + load_vec(skip, v_is_f32, c / vdim) * x[(size_t)t * x_stride + c];
        v *= g / (1.f + expf(-g));
        row[i] = v;
        ss += v * v;
    }
    const float r = rsqrtf(block_sum(ss, red) / (float)len + eps);
    for (int i = threadIdx.x; i < len; i += blockDim.x)
        out[(size_t)t * inner + c0 + i] = Cvt<T>::from_f32(row[i] * r * load_vec(norm_w, v_is_f32, c0 + i));
}

template <typename T>
static int launch_conv(const void* src, int row_stride, int col0, float* state, const void* w, const void* bias, int w_is_f32,
                       float* out, const int* tok_seq, const int* cu_q, const int* seq_slot, int T_, int B, int C, int taps,
                       cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (taps < 1 || taps > MB_MAX_TAPS || C <= 0) return RF_ERR_UNSUPPORTED;
    const bool groups_of_four = C % 4 == 0 && col0 % 4 == 0 && row_stride % 4 == 0 && taps <= 4 &&
                                (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(state) & 15) == 0;
    if (groups_of_four && T_ >= 64) {
        const dim3 grid((T_ + CV_TOK - 1) / CV_TOK, (C / 4 + 255) / 256);
#define CONV_VEC(TAPS) rf_launch(conv_silu_vec_kernel<T, TAPS>, grid, dim3(256), 0, st, reinterpret_cast<const T*>(src), row_stride, \
                                 col0, (const float*)state, w, bias, w_is_f32, out, tok_seq, cu_q, seq_slot, C, T_)
        if (taps == 1) CONV_VEC(1); else if (taps == 2) CONV_VEC(2); else if (taps == 3) CONV_VEC(3); else CONV_VEC(4);
#undef CONV_VEC
        RF_LAUNCH_CHECK();
    } else {
    int by = T_ >= 296 ? 1 : (C + 255) / 256;
    if (by > 64) by = 64;
    rf_launch(conv_silu_kernel<T>, dim3(T_, by), dim3(256), 0, st, reinterpret_cast<const T*>(src), row_stride, col0,
              (const float*)state, w, bias, w_is_f32, out, tok_seq, cu_q, seq_slot, C, taps);
    RF_LAUNCH_CHECK();
    }
    if (taps > 1) {
        int cy = (C + 255) / 256;
        if (cy > 64) cy = 64;
        rf_launch(conv_state_update_kernel<T>, dim3(B, cy), dim3(256), 0, st, reinterpret_cast<const T*>(src), row_stride, col0,
                  state, cu_q, seq_slot, C, taps);
        RF_LAUNCH_CHECK();
    }
    return 0;
}

template <typename T>
static int launch_finish(const float* y, const float* x, int x_stride, const void* gate, int gate_stride, const void* skip,
                         const void* norm_w, int v_is_f32, void* out, int T_, int inner, int parts, int vdim, float eps,
                         cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (parts < 1 || inner % parts || vdim < 1 || parts > 65535) return RF_ERR_BAD_ARG;
    const size_t smem = (size_t)(inner / parts + 34) * sizeof(float);
    if (smem > 48 * 1024) return RF_ERR_UNSUPPORTED;
    rf_launch(mamba_finish_kernel<T>, dim3(T_, parts), dim3(256), smem, st, y, x, x_stride, reinterpret_cast<const T*>(gate),
              gate_stride, skip, norm_w, v_is_f32, reinterpret_cast<T*>(out), inner, parts, vdim, eps);
    RF_LAUNCH_CHECK();
    return 0;
}

extern "C" {
// dtype: 0 = float32, 1 = bfloat16 (of the projection's output).  src [T, row_stride], the convolution's C channels from
// column col0 on; state float [slots, taps-1, C], read and then replaced by the step's last inputs; w [C, taps] and bias
// [C] of one dtype (w_is_f32, else bfloat16); out float [T, C].
int rf_conv_silu(int dtype, const void* src, int row_stride, int col0, float* state, const void* w, const void* bias,
                 int w_is_f32, float* out, const int* tok_seq, const int* cu_q, const int* seq_slot, int T_, int B, int C,
                 int taps, cudaStream_t st) {
    return dtype == 0 ? launch_conv<float>(src, row_stride, col0, state, w, bias, w_is_f32, out, tok_seq, cu_q, seq_slot, T_, B, C, taps, st)
                      : launch_conv<__nv_bfloat16>(src, row_stride, col0, state, w, bias, w_is_f32, out, tok_seq, cu_q, seq_slot, T_, B, C, taps, st);
}
// z float [T, heads]; dt_bias, a_log [heads] of one dtype; ab float [T, heads, 2]
int rf_mamba_gates(const float* z, const void* dt_bias, const void* a_log, int v_is_f32, float* ab, int T_, int heads,
                   cudaStream_t st) {
    const size_t n = (size_t)T_ * heads;
    if (n == 0) return 0;
    const size_t blocks = (n + 255) / 256;
    rf_launch(mamba_gates_kernel, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st, z, dt_bias, a_log,
              v_is_f32, ab, heads, n);
    RF_LAUNCH_CHECK();
    return 0;
}
// dtype of gate and out; skip [inner / vdim] (one per head), norm_w [inner], of one dtype (v_is_f32, else bfloat16)
int rf_mamba_finish(int dtype, const float* y, const float* x, int x_stride, const void* gate, int gate_stride,
                    const void* skip, const void* norm_w, int v_is_f32, void* out, int T_, int inner, int parts, int vdim,
                    float eps, cudaStream_t st) {
    return dtype == 0 ? launch_finish<float>(y, x, x_stride, gate, gate_stride, skip, norm_w, v_is_f32, out, T_, inner, parts, vdim, eps, st)
                      : launch_finish<__nv_bfloat16>(y, x, x_stride, gate, gate_stride, skip, norm_w, v_is_f32, out, T_, inner, parts, vdim, eps, st);
}
}
