// Routing of a mixture of experts: which experts a token uses, with what weights, and the tokens sorted by expert
// so that one grouped product serves all experts of a step without the host ever learning the counts.
//
//   moe_route     per token: the `top` largest of E router logits (32-bit; of equal logits the lower index), and
//                 their weights: the softmax over the chosen logits only (scoring 0), or each chosen logit's own
//                 sigmoid, not renormalised (scoring 1), or each chosen logit's share of the softmax over all E
//                 logits, not renormalised (scoring 2)
//   moe_sort      counting sort of the T*top (token, choice) pairs by expert: perm[sorted row] = pair,
//                 inv[pair] = sorted row, and the table of row tiles for the grouped product
//                 (tiles[0] = number of tiles, then (expert, first row, end row) per tile; a tile never spans experts)
//   moe_combine   out[t] = sum over the token's choices, in the order of the choices, of weight * expert output row
//                 (no weights: the plain sum, for designs whose weights went into the experts' inputs)
//   (moe_sort can also leave the pairs' weights in the order of the sorted rows, for designs that weight an expert's input)
// A row of the grouped product depends on its own token alone, so where the sort puts a pair changes no bit.
#include "common.cuh"

#define MOE_MAX_TOP 16

__global__ void moe_route_kernel(const float* __restrict__ logits, int E, int top, int* __restrict__ idx,
                                 float* __restrict__ w, int T_, int scoring) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T_) return;
    const float* z = logits + (size_t)t * E;
    int chosen[MOE_MAX_TOP];
    float val[MOE_MAX_TOP];
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e) {
            bool taken = false;
            for (int c = 0; c < k; ++c) taken |= chosen[c] == e;
            const float v = z[e];
            if (!taken && (best < 0 || v > bv)) { best = e; bv = v; }
        }
        chosen[k] = best;
        val[k] = bv;
    }
    if (scoring == 2) {                              // the chosen experts' shares of the softmax over ALL experts
        float largest = -INFINITY, sum = 0.f;
        for (int e = 0; e < E; ++e) largest = fmaxf(largest, z[e]);
        for (int e = 0; e < E; ++e) sum += expf(z[e] - largest);
        for (int k = 0; k < top; ++k) {
            idx[(size_t)t * top + k] = chosen[k];
            w[(size_t)t * top + k] = expf(val[k] - largest) / sum;
        }
        return;
    }
    if (scoring == 1) {
        for (int k = 0; k < top; ++k) {
            idx[(size_t)t * top + k] = chosen[k];
            w[(size_t)t * top + k] = 1.f / (1.f + expf(-val[k]));
        }
        return;
    }
    float sum = 0.f;
    const float largest = val[0];
    for (int k = 0; k < top; ++k) { val[k] = expf(val[k] - largest); sum += val[k]; }
    for (int k = 0; k < top; ++k) {
        idx[(size_t)t * top + k] = chosen[k];
        w[(size_t)t * top + k] = val[k] / sum;
    }
}

// One block.  counts/cursors live in shared memory (E <= 1024).
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int n, int E, int BM, int* __restrict__ perm, int* __restrict__ inv,
                int* __restrict__ offsets, int* __restrict__ tiles, int max_tiles, const float* __restrict__ w,
                float* __restrict__ w_sorted) {
    __shared__ int counts[1024];
    __shared__ int cursor[1024];
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = off;
            cursor[e] = off;
            for (int r = off; r < off + counts[e] && nt < max_tiles; r += BM) {
                tiles[1 + 3 * nt] = e;
                tiles[2 + 3 * nt] = r;
                tiles[3 + 3 * nt] = min(r + BM, off + counts[e]);
                ++nt;
            }
            off += counts[e];
        }
        offsets[E] = off;
        tiles[0] = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int r = atomicAdd(&cursor[idx[i]], 1);
        perm[r] = i;
        inv[i] = r;
        if (w_sorted != nullptr) w_sorted[r] = w[i];     // the pairs' weights in sorted order, for a product that reads them by row
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ inv, const float* __restrict__ w,
                                   float* __restrict__ out, int top, int H, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / H, c = i - t * H;
        float acc = 0.f;
        for (int k = 0; k < top; ++k) acc = fmaf(w != nullptr ? w[t * top + k] : 1.f, y[(size_t)inv[t * top + k] * H + c], acc);
        out[i] = acc;
    }
}

// out[r, :] = x[perm[r] / top, :]: the activations in the sorted order, for a grouped product that reads whole tiles
// of rows (elem_bytes per element; rows are copied 16 bytes at a time where they are aligned for it)
__global__ void moe_gather_kernel(const uint8_t* __restrict__ x, long long x_stride_bytes, const int* __restrict__ perm,
                                  int top, uint8_t* __restrict__ out, int row_bytes, int vec) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const uint8_t* src = x + (size_t)(perm[r] / top) * x_stride_bytes;
    uint8_t* dst = out + (size_t)r * row_bytes;
    if (vec) {
        for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = src[i];
    }
}

extern "C" {
int rf_moe_gather(const void* x, long long x_stride_bytes, const int* perm, int top, void* out, int row_bytes, int n,
                  cudaStream_t st) {
    if (n <= 0 || row_bytes <= 0) return 0;
    const int vec = row_bytes % 16 == 0 && x_stride_bytes % 16 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                    !(reinterpret_cast<uintptr_t>(out) & 15);
    rf_launch(moe_gather_kernel, dim3(n), dim3(128), 0, st, reinterpret_cast<const uint8_t*>(x), x_stride_bytes, perm, top,
              reinterpret_cast<uint8_t*>(out), row_bytes, vec);
    RF_LAUNCH_CHECK();
    return 0;
}
static int route(const float* logits, int E, int top, int* idx, float* w, int T_, int scoring, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP || top > E) return RF_ERR_UNSUPPORTED;
    if (scoring < 0 || scoring > 2) return RF_ERR_BAD_ARG;
    rf_launch(moe_route_kernel, dim3((T_ + 127) / 128), dim3(128), 0, st, logits, E, top, idx, w, T_, scoring);
    RF_LAUNCH_CHECK();
    return 0;
}
int rf_moe_route(const float* logits, int E, int top, int* idx, float* w, int T_, cudaStream_t st) {
    return route(logits, E, top, idx, w, T_, 0, st);
}
// scoring: 0 = softmax over the chosen logits, 1 = sigmoid of each chosen logit, 2 = share of the softmax over all logits
int rf_moe_route_scored(const float* logits, int E, int top, int* idx, float* w, int T_, int scoring, cudaStream_t st) {
    return route(logits, E, top, idx, w, T_, scoring, st);
}
static int sort_pairs(const int* idx, int n, int E, int BM, int* perm, int* inv, int* offsets, int* tiles, int max_tiles,
                      const float* w, float* w_sorted, cudaStream_t st) {
    if (n <= 0) return 0;
    if (E < 1 || E > 1024 || BM < 1 || ((w == nullptr) != (w_sorted == nullptr))) return RF_ERR_UNSUPPORTED;
    rf_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, st, idx, n, E, BM, perm, inv, offsets, tiles, max_tiles, w, w_sorted);
    RF_LAUNCH_CHECK();
    return 0;
}
int rf_moe_sort(const int* idx, int n, int E, int BM, int* perm, int* inv, int* offsets, int* tiles, int max_tiles,
                cudaStream_t st) {
    return sort_pairs(idx, n, E, BM, perm, inv, offsets, tiles, max_tiles, nullptr, nullptr, st);
}
// The same, and w_sorted[r] = w[perm[r]] (float [n]): the pairs' weights in the order of the sorted rows.
int rf_moe_sort_w(const int* idx, int n, int E, int BM, int* perm, int* inv, int* offsets, int* tiles, int max_tiles,
                  const float* w, float* w_sorted, cudaStream_t st) {
    return sort_pairs(idx, n, E, BM, perm, inv, offsets, tiles, max_tiles, w, w_sorted, st);
}
int rf_moe_combine(const float* y, const int* inv, const float* w, float* out, int top, int H, int T_, cudaStream_t st) {
    const size_t n = (size_t)T_ * H;
    if (n == 0) return 0;
    const size_t blocks = (n + 255) / 256;
    rf_launch(moe_combine_kernel, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st, y, inv, w, out, top, H, n);
    RF_LAUNCH_CHECK();
    return 0;
}
}
