// Embedding gather, residual-add + RMSNorm, rotary position encoding fused with the
// cache write, and SwiGLU.  Each kernel is templated on the compute dtype (float for
// the true 32-bit path, bfloat16 for serving); the residual stream is 32-bit in both.
//
// What they compute follows maeddesg/ROCmForge's hip_kernels/norm.hip:18-84 (RMSNorm),
// rope.hip:48-91 and attention.hip:1561-1621 (NeoX rotation fused with the cache
// write), elementwise.hip:72-82 (SiLU, multiply) and the embedding gathers of
// elementwise.hip:243-445; how they are launched and laid out is this library's own.
#include "common.cuh"

// Four neighbouring elements as one access.
template <typename T> struct Four;
template <> struct Four<float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Four<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
        v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<const uint32_t*>(&a); x.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] widened to 32-bit (the residual stream).
// With pos_table (a learned vector per position, [P, H]) row tok_pos[t] of it is added, in 32-bit; with rounded, the
// stream's row is also left there in the table's dtype (for sub-layers that read the stream itself).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int H, int V, const T* __restrict__ pos_table,
                             const int* __restrict__ tok_pos, int P, T* __restrict__ rounded, float scale) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);   // ids are validated on the host; never read outside
    const T* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    if (pos_table != nullptr || rounded != nullptr) {
        int ps = pos_table != nullptr ? tok_pos[t] : 0;
        ps = ps < 0 ? 0 : (ps >= P ? P - 1 : ps);       // the cache refuses sequences longer than the table
        const T* prow = pos_table != nullptr ? pos_table + (size_t)ps * H : nullptr;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = Cvt<T>::to_f32(row[i]) * scale + (prow != nullptr ? Cvt<T>::to_f32(prow[i]) : 0.f);
            o[i] = v;
            if (rounded != nullptr) rounded[(size_t)t * H + i] = Cvt<T>::from_f32(v);
        }
        return;
    }
    // four elements per access where rows allow it: a decode step starts with this kernel, and 14 rounds of 2-byte
    // loads from a table row that lies in DRAM took 10 us
    if (H % 4 == 0 && (reinterpret_cast<uintptr_t>(table) % (4 * sizeof(T))) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        for (int i = 4 * threadIdx.x; i < H; i += 4 * blockDim.x) {
            float v[4];
            Four<T>::load(row + i, v);
            *reinterpret_cast<float4*>(o + i) = make_float4(v[0] * scale, v[1] * scale, v[2] * scale, v[3] * scale);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = Cvt<T>::to_f32(row[i]) * scale;
}

// ---------------------------------------------------------------- add + RMSNorm
// v = h[row] + sum_s pending[s][row];  y = v * rsqrt(mean(v^2) + eps) * w.
// pending_kind: 0 none, 1 = n_pending 32-bit partial sums [S, T, H] (split-K outputs,
// added in index order), 2 = one [T, H] tensor in the compute dtype.
// rows == nullptr: one block per token, h is updated in place.
// rows != nullptr: block r reads token rows[r], writes y[r] and leaves h alone.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const void* __restrict__ pending,
                                   int pending_kind, int n_pending, size_t pending_stride,
                                   const void* __restrict__ w, int w_is_f32, float eps,
                                   T* __restrict__ y, const int* __restrict__ rows, int H) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row_buf[];          // H floats + 33 for the reduction
    float* red = row_buf + H;
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float* hrow = h + (size_t)t * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hrow[i];
        if (pending_kind == 1) {
            const float* p = reinterpret_cast<const float*>(pending) + (size_t)t * H + i;
            for (int s = 0; s < n_pending; ++s) v += p[(size_t)s * pending_stride];
        } else if (pending_kind == 2) {
            v += Cvt<T>::to_f32(reinterpret_cast<const T*>(pending)[(size_t)t * H + i]);
        }
        row_buf[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    T* yrow = y + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = row_buf[i];
        if (!rows && pending_kind != 0) hrow[i] = v;
        yrow[i] = Cvt<T>::from_f32(v * inv * load_vec(w, w_is_f32, i));
    }
}

// The same for rows whose length is a multiple of 4: the row lives in registers (at most NV float4 per
// thread), every load is 16 bytes wide and independent of the others, so a short row costs a few
// memory round trips instead of a chain of them.  Sums are formed in the same order as above
// (h first, then the partial sums in index order), element by element.
//
// A row may be shared by a thread-block cluster of `cl` CTAs (few rows: a decode step's norm reads the K-split
// partial sums of the product before it, 150 KB a row at width 3,584 with ten splits, and one CTA per row leaves a
// handful of SMs pulling all of that from L2).  The CTAs' threads are numbered through (rank * blockDim + thread)
// and work exactly as the threads of one large block would; the warps' sums of squares are pushed into every
// CTA's shared memory and folded by the same tree as in block_sum, so the result is bit for bit that of one CTA.
// The pushes are st.async stores that report their bytes to the receiving CTA's mbarrier, set up before the cluster's
// one barrier at the kernel's top (which the dependency wait hides): a CTA waits for the words it expects and for
// nothing else.  With plain remote stores and a second cluster barrier (arrive.release, wait.acquire) behind them
// the exchange cost 0.9 us of a kernel that otherwise takes 1.3 (a decode step of the 7B shape at batch 8 2.59 -> 2.54
// ms, at batch 1 2.51 -> 2.45 ms).  The wait is bounded: status 7 when a peer's words never come.
__device__ __forceinline__ float cluster_block_sum(float v, float* red, uint64_t* bar, int vt, int n_warps, int cl,
                                                    int* status) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // every peer has started and set up its barrier
    if (lane == 0) {
        // a warp's sum goes into every CTA's array by a store that reports its bytes to that CTA's mbarrier: a CTA
        // then waits for the words it expects and for nothing else (no second cluster barrier, no release fence)
        const uint32_t mine = (uint32_t)__cvta_generic_to_shared(&red[vt >> 5]);
        const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
        for (int r = 0; r < cl; ++r) {
            uint32_t remote, remote_bar;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(r));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(mbar), "r"(r));
            asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                         ::"r"(remote), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
        }
    }
    {
        const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(bar);
        uint32_t ok = 0;
        unsigned long long t0 = 0;
        for (long long it = 0; !ok; ++it) {
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(mbar), "r"(0u) : "memory");
            if (ok) break;
            if ((it & 63) == 63) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > 2000000000ull) break;     // 2 s: a peer's words never came; the row is invalid
            }
        }
        if (!ok && threadIdx.x == 0 && status) atomicExch(status, 7);
    }
    if (warp == 0) {
        float t = lane < n_warps ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// INF: partial sums of one element group asked for at once.  A decode step's norm is a chain of L2 round trips and
// nothing else; ten or fifteen K splits read four at a time (and the rest one by one) were four to six trips, sixteen at
// a time they are one.  The wide form needs its registers: it is compiled for blocks of at most 256 threads.
template <typename T, int NV, int INF, int MAXT>
__global__ void __launch_bounds__(MAXT)
add_rmsnorm_vec_kernel(float* __restrict__ h, const void* __restrict__ pending, int pending_kind, int n_pending,
                       size_t pending_stride, const void* __restrict__ w, int w_is_f32, float eps,
                       T* __restrict__ y, const int* __restrict__ rows, int H, int cl, int* __restrict__ status) {
    pdl_trigger();
    __shared__ float red[34];
    __shared__ __align__(8) uint64_t sum_bar;
    if (cl > 1) {
        if (threadIdx.x == 0) {                          // this CTA expects a word from every warp of the row's cluster
            const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(&sum_bar);
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(mbar));
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"((uint32_t)(cl * blockDim.x / 32 * 4)) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");            // "started": peers may store here
    }
    const int r = blockIdx.x / cl;
    const int t = rows ? rows[r] : r;
    const int nvec = H >> 2;
    int rank = 0;
    if (cl > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int vt = rank * blockDim.x + threadIdx.x, VT = cl * blockDim.x;       // this thread among the row's threads
    uint4 wraw[NV];                              // the norm's weights (four floats, or four bfloat16 in x and y):
#pragma unroll                                   // no kernel writes them, so they are fetched while the kernel
    for (int i = 0; i < NV; ++i) {               // before this one still runs
        const int c = vt + i * VT;
        wraw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (c < nvec) {
            if (w_is_f32) {
                wraw[i] = reinterpret_cast<const uint4*>(w)[c];
            } else {
                const uint2 two = reinterpret_cast<const uint2*>(w)[c];
                wraw[i].x = two.x; wraw[i].y = two.y;
            }
        }
    }
    pdl_wait();
    float4* hrow = reinterpret_cast<float4*>(h + (size_t)t * H);
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = vt + i * VT;
        if (c < nvec) {
            float4 a = hrow[c];
            if (pending_kind == 1) {
                const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(pending) + (size_t)t * H) + c;
                if constexpr (INF > 4) {
                    for (int s2 = 0; s2 < n_pending; s2 += INF) {    // INF loads in flight, added in index order
                        float4 b[INF];
#pragma unroll
                        for (int u = 0; u < INF; ++u)
                            if (s2 + u < n_pending)
                                b[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + (size_t)(s2 + u) * pending_stride);
#pragma unroll
                        for (int u = 0; u < INF; ++u)
                            if (s2 + u < n_pending) { a.x += b[u].x; a.y += b[u].y; a.z += b[u].z; a.w += b[u].w; }
                    }
                } else {
                    int s2 = 0;
                    for (; s2 + 4 <= n_pending; s2 += 4) {   // four loads in flight, added in index order
                        float4 b[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            b[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + (size_t)(s2 + u) * pending_stride);
#pragma unroll
                        for (int u = 0; u < 4; ++u) { a.x += b[u].x; a.y += b[u].y; a.z += b[u].z; a.w += b[u].w; }
                    }
                    for (; s2 < n_pending; ++s2) {
                        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + (size_t)s2 * pending_stride);
                        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                    }
                }
            } else if (pending_kind == 2) {
                const T* p = reinterpret_cast<const T*>(pending) + (size_t)t * H + 4 * c;
                a.x += Cvt<T>::to_f32(p[0]); a.y += Cvt<T>::to_f32(p[1]);
                a.z += Cvt<T>::to_f32(p[2]); a.w += Cvt<T>::to_f32(p[3]);
            }
            v[i] = a;
            ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        }
    }
    const float total = cl > 1 ? cluster_block_sum(ss, red, &sum_bar, vt, VT >> 5, cl, status) : block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    T* yrow = y + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = vt + i * VT;
        if (c < nvec) {
            if (!rows && pending_kind != 0) hrow[c] = v[i];
            float w0, w1, w2, w3;
            if (w_is_f32) {
                w0 = __uint_as_float(wraw[i].x); w1 = __uint_as_float(wraw[i].y);
                w2 = __uint_as_float(wraw[i].z); w3 = __uint_as_float(wraw[i].w);
            } else {                             // a bfloat16 is the upper half of a float
                w0 = __uint_as_float(wraw[i].x << 16); w1 = __uint_as_float(wraw[i].x & 0xffff0000u);
                w2 = __uint_as_float(wraw[i].y << 16); w3 = __uint_as_float(wraw[i].y & 0xffff0000u);
            }
            const float o0 = v[i].x * inv * w0, o1 = v[i].y * inv * w1;
            const float o2 = v[i].z * inv * w2, o3 = v[i].w * inv * w3;
            const float ov[4] = {o0, o1, o2, o3};
            Four<T>::store(yrow + 4 * c, ov);              // one 16-byte (8-byte) store: the row is aligned for it
        }
    }
}

// The norm of many rows without a pending update (a prompt step: the products add into the stream themselves).  The
// kernel above keeps a row in registers, and 56 registers a thread leave room for four rows per SM: 56 KB in flight,
// which one L2 round trip turns into 4 TB/s over the GPU (12 us for 2,048 rows of 3,584).  Here a row is read twice,
// the second time from L1 (8 rows of 14 KB per SM fit it), so a thread needs 20-odd registers, eight CTAs share an SM
// and twice the bytes are in flight.  Same sums in the same order as above (block_sum over one float4 per step).
template <typename T>
__global__ void __launch_bounds__(256, 8)
rmsnorm_rows_kernel(const float* __restrict__ h, const void* __restrict__ w, int w_is_f32, float eps, T* __restrict__ y,
                    int H) {
    pdl_trigger();
    __shared__ float red[34];
    const int r = blockIdx.x, nvec = H >> 2;
    pdl_wait();
    const float4* hrow = reinterpret_cast<const float4*>(h + (size_t)r * H);
    float ss = 0.f;
    for (int c0 = threadIdx.x; c0 < nvec; c0 += 4 * blockDim.x) {          // four loads in flight per thread
        float4 a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + i * blockDim.x;
            a[i] = c < nvec ? hrow[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += a[i].x * a[i].x + a[i].y * a[i].y + a[i].z * a[i].z + a[i].w * a[i].w;
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    T* yrow = y + (size_t)r * H;
#pragma unroll 4
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
        const float4 a = hrow[c];
        float w0, w1, w2, w3;
        if (w_is_f32) {
            const float4 t = reinterpret_cast<const float4*>(w)[c];
            w0 = t.x; w1 = t.y; w2 = t.z; w3 = t.w;
        } else {                                 // a bfloat16 is the upper half of a float
            const uint2 two = reinterpret_cast<const uint2*>(w)[c];
            w0 = __uint_as_float(two.x << 16); w1 = __uint_as_float(two.x & 0xffff0000u);
            w2 = __uint_as_float(two.y << 16); w3 = __uint_as_float(two.y & 0xffff0000u);
        }
        const float ov[4] = {a.x * inv * w0, a.y * inv * w1, a.z * inv * w2, a.w * inv * w3};
        Four<T>::store(yrow + 4 * c, ov);
    }
}

// ---------------------------------------------------------------- rotation + cache write
// Rows of q | k | v, [T, (nh + 2*nkv) * hd], come either in the compute dtype (src, one tensor)
// or as n_partials 32-bit partial sums of a K-split product plus a bias (the sum is formed here,
// in index order).  q is rotated and written to q_out (which may be the source itself); k is
// rotated and v copied into the page of (slot, position): pages are [n_pages, nkv, RF_PAGE, hd].
// The angle is float(pos) * inv_freq[i] in 32-bit; sincosf is the accurate one.
template <typename T, bool PARTIALS>
__global__ void rope_kv_write_kernel(const void* __restrict__ src, int row_stride, int n_partials,
                                     size_t partial_stride, const void* __restrict__ bias, int bias_is_f32,
                                     T* __restrict__ q_out, int q_out_stride, int nh, int nkv, int hd,
                                     const float* __restrict__ inv_freq,
                                     const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                     const int* __restrict__ seq_slot,
                                     const int* __restrict__ block_table, int max_pages,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages, int write_kv,
                                     int rot_dim, int interleaved) {
    // grid: (token, block of pairs).  Pair index space: nh + nkv rotated heads, then nkv value heads,
    // hd/2 pairs each (a value "pair" is two neighbouring elements, copied).
    // Position, slot, page, frequency, bias and the angle's sine and cosine do not depend on the kernel
    // before this one (no kernel of a step writes them): all of that is done before pdl_wait(), so that
    // after it only the loads of the product's sums and the stores remain.
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;
    const int n_pairs = (nh + 2 * nkv) * half;
    if (idx >= n_pairs) return;
    const int head = idx / half, i = idx - head * half;
    if (head >= nh && !write_kv) return;
    const int pos = tok_pos[t];
    // which two elements of the head this pair is, and whether they turn: the first rot_dim elements of a query or
    // key head are rotated, as pairs (i, i + rot_dim/2) or (2i, 2i+1); the rest, and values, pass through
    const int rh = rot_dim >> 1;
    bool rotated = head < nh + nkv;
    int e0, e1;
    if (rotated && interleaved) { e0 = 2 * i; e1 = e0 + 1; rotated = e0 < rot_dim; }
    else if (rotated && i < rh) { e0 = i; e1 = i + rh; }
    else if (rotated) { e0 = rot_dim + 2 * (i - rh); e1 = e0 + 1; rotated = false; }
    else { e0 = 2 * i; e1 = e0 + 1; }
    const int col0 = head * hd + e0, col1 = head * hd + e1;
    float b0 = 0.f, b1 = 0.f;
    if (PARTIALS && bias) { b0 = load_vec(bias, bias_is_f32, col0); b1 = load_vec(bias, bias_is_f32, col1); }
    size_t page_base = 0;
    if (head >= nh) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = block_table[(size_t)slot * max_pages + pos / RF_PAGE];
        page_base = (size_t)page * nkv * RF_PAGE * hd + (size_t)(pos % RF_PAGE) * hd;
    }
    float s = 0.f, c = 1.f;
    if (rotated) sincosf((float)pos * inv_freq[i], &s, &c);
    pdl_wait();
    float x0, x1;
    if (PARTIALS) {
        const float* p = reinterpret_cast<const float*>(src) + (size_t)t * row_stride;
        x0 = b0; x1 = b1;
        for (int sp = 0; sp < n_partials; sp += 8) {    // eight pairs of loads in flight at once, added in index order
            float u0[8], u1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (sp + u < n_partials) {
                    u0[u] = p[(size_t)(sp + u) * partial_stride + col0];
                    u1[u] = p[(size_t)(sp + u) * partial_stride + col1];
                }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (sp + u < n_partials) { x0 += u0[u]; x1 += u1[u]; }
        }
    } else {
        x0 = Cvt<T>::to_f32(reinterpret_cast<const T*>(src)[(size_t)t * row_stride + col0]);
        x1 = Cvt<T>::to_f32(reinterpret_cast<const T*>(src)[(size_t)t * row_stride + col1]);
    }
    if (rotated) {
        const float r0 = x0 * c - x1 * s, r1 = x0 * s + x1 * c;
        x0 = r0; x1 = r1;
    }
    T* dst = head < nh ? q_out + (size_t)t * q_out_stride + (size_t)head * hd
           : head < nh + nkv ? k_pages + page_base + (size_t)(head - nh) * RF_PAGE * hd
                             : v_pages + page_base + (size_t)(head - nh - nkv) * RF_PAGE * hd;
    dst[e0] = Cvt<T>::from_f32(x0);
    dst[e1] = Cvt<T>::from_f32(x1);
}

// The same for many tokens (prompts) whose q | k | v rows are one tensor in the compute dtype: a block per
// token; a thread takes four neighbouring pair indices, computes their sines and cosines once and walks
// over the heads in steps of blockDim.x / (hd/8) with loads and stores of four elements, so the
// trigonometry is shared by the heads and every access is 8 or 16 bytes wide.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_rows_kernel(const T* __restrict__ src, int row_stride, T* __restrict__ q_out, int q_out_stride,
                          int nh, int nkv, int hd, const float* __restrict__ inv_freq,
                          const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                          const int* __restrict__ seq_slot, const int* __restrict__ block_table, int max_pages,
                          T* __restrict__ k_pages, T* __restrict__ v_pages, int write_kv) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = hd >> 1, groups = half >> 2;        // groups of four pairs per head
    const int g = threadIdx.x % groups, lane_head = threadIdx.x / groups, head_step = blockDim.x / groups;
    if (lane_head >= head_step) return;                  // threads beyond the last whole row of groups
    const int pos = tok_pos[t];
    size_t page_base = 0;
    if (write_kv) {
        const int slot = seq_slot[tok_seq[t]];
        const int page = block_table[(size_t)slot * max_pages + pos / RF_PAGE];
        page_base = (size_t)page * nkv * RF_PAGE * hd + (size_t)(pos % RF_PAGE) * hd;
    }
    float sn[4], cs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) sincosf((float)pos * inv_freq[4 * g + j], &sn[j], &cs[j]);
    pdl_wait();
    const T* row = src + (size_t)t * row_stride;
    const int rotated = write_kv ? nh + nkv : nh;
    for (int head = lane_head; head < rotated; head += head_step) {
        float x0[4], x1[4], r0[4], r1[4];
        Four<T>::load(row + (size_t)head * hd + 4 * g, x0);
        Four<T>::load(row + (size_t)head * hd + half + 4 * g, x1);
#pragma unroll
        for (int j = 0; j < 4; ++j) { r0[j] = x0[j] * cs[j] - x1[j] * sn[j]; r1[j] = x0[j] * sn[j] + x1[j] * cs[j]; }
        T* dst = head < nh ? q_out + (size_t)t * q_out_stride + (size_t)head * hd
                           : k_pages + page_base + (size_t)(head - nh) * RF_PAGE * hd;
        Four<T>::store(dst + 4 * g, r0);
        Four<T>::store(dst + half + 4 * g, r1);
    }
    if (write_kv)
        for (int vh = lane_head; vh < nkv; vh += head_step) {
            float a[4], b[4];
            const T* sv = row + (size_t)(nh + nkv + vh) * hd;
            Four<T>::load(sv + 4 * g, a);
            Four<T>::load(sv + half + 4 * g, b);
            T* dst = v_pages + page_base + (size_t)vh * RF_PAGE * hd;
            Four<T>::store(dst + 4 * g, a);
            Four<T>::store(dst + half + 4 * g, b);
        }
}

// ---------------------------------------------------------------- SwiGLU
// gu: [T, 2I] with gate_j at column 2j and up_j at column 2j+1 (the fused weight is
// interleaved row by row at load time); a[t, j] = silu(gate) * up, evaluated in 32-bit.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ a, size_t n_out, int I) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_out;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, j = idx - t * I;
        const float g = Cvt<T>::to_f32(gu[t * 2 * I + 2 * j]);
        const float u = Cvt<T>::to_f32(gu[t * 2 * I + 2 * j + 1]);
        a[idx] = Cvt<T>::from_f32(g / (1.f + expf(-g)) * u);
    }
}

// ---------------------------------------------------------------- squared ReLU
// a = max(x, 0)^2, evaluated in 32-bit.
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ a, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(Cvt<T>::to_f32(x[idx]), 0.f);
        a[idx] = Cvt<T>::from_f32(v * v);
    }
}

// ---------------------------------------------------------------- a row vector added to every row of the stream
template <typename T>
__global__ void add_row_kernel(float* __restrict__ h, const T* __restrict__ vec, size_t n, int H) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x)
        h[idx] += Cvt<T>::to_f32(vec[idx % H]);
}

// ---------------------------------------------------------------- a normed branch added into the stream
// The residual update of a block that norms its sub-layers' outputs as well as their inputs, all in 32-bit:
//   m = a0                                            (one branch), or
//   m = (rms(a0) * w0 + rms(a1) * w1) / 2             (two branches side by side, each normed with its own weight)
//   h += rms(m) * w_post (+ extra)                    (extra: a row vector that the schedule adds before the next layer)
//   y_next = rms(h) * w_next in the compute dtype     (the norm that reads the stream next, if the caller knows it;
//                                                      y_next without w_next: h itself, rounded to the compute dtype)
// with rms(x) = x / sqrt(mean(x^2) + eps).  A branch comes as n0 (n1) partial sums [n][rows][H] of a K-split product,
// added here in index order.  A block per row; the rows stay in shared memory between the passes.
template <typename T>
__global__ void __launch_bounds__(1024)
branch_norm_add_kernel(float* __restrict__ h, const float* __restrict__ a0, int n0, const void* __restrict__ w0,
                       const float* __restrict__ a1, int n1, size_t part_stride, const void* __restrict__ w1,
                       const void* __restrict__ w_post, const void* __restrict__ extra, const void* __restrict__ w_next,
                       T* __restrict__ y_next, int w_is_f32, float eps, int H) {
    extern __shared__ float row[];                  // [H], a second [H] for the other branch, 34 for the sums
    float* other = row + H;
    float* red = other + H;
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * H;
    const float invH = 1.f / (float)H;
    pdl_wait();
    if (a1 != nullptr) {
        float s0 = 0.f, s1 = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float x = 0.f, z = 0.f;
#pragma unroll 4
            for (int s = 0; s < n0; ++s) x += a0[(size_t)s * part_stride + base + c];
#pragma unroll 4
            for (int s = 0; s < n1; ++s) z += a1[(size_t)s * part_stride + base + c];
            row[c] = x; other[c] = z;
            s0 += x * x; s1 += z * z;
        }
        const float r0 = rsqrtf(block_sum(s0, red) * invH + eps);
        const float r1 = rsqrtf(block_sum(s1, red) * invH + eps);
        for (int c = threadIdx.x; c < H; c += blockDim.x)
            row[c] = 0.5f * (row[c] * r0 * load_vec(w0, w_is_f32, c) + other[c] * r1 * load_vec(w1, w_is_f32, c));
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float x = 0.f;
#pragma unroll 4
            for (int s = 0; s < n0; ++s) x += a0[(size_t)s * part_stride + base + c];
            row[c] = x;
        }
    }
    float sm = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) sm += row[c] * row[c];      // a thread reads what it wrote
    const float rm = rsqrtf(block_sum(sm, red) * invH + eps);
    float sh = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = h[base + c] + row[c] * rm * load_vec(w_post, w_is_f32, c);
        if (extra != nullptr) v += load_vec(extra, w_is_f32, c);
        h[base + c] = v;
        row[c] = v;
        sh += v * v;
    }
    if (y_next == nullptr) return;
    if (w_next == nullptr) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) y_next[base + c] = Cvt<T>::from_f32(row[c]);
        return;
    }
    const float rh = rsqrtf(block_sum(sh, red) * invH + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        y_next[base + c] = Cvt<T>::from_f32(row[c] * rh * load_vec(w_next, w_is_f32, c));
}

// ---------------------------------------------------------------- per-head unit norm + rotation + cache write
// A warp per head of a token's q | k | v row: q heads and k heads have hd elements, v heads hdv.  The row comes in
// the compute dtype or as n_partials 32-bit partial sums.  With unit_norm every q and k head is divided by its root
// mean square (x / sqrt(mean(x^2) + eps), 32-bit) and, if q_norm_w / k_norm_w are given ([hd], one weight vector for
// all query heads and one for all key heads), multiplied by it; then the first rot_dim elements turn as in the kernel
// above (rot_dim 0: none); q goes to q_out, k and v into the page of (slot, position).  Key pages are
// [n_pages, nkv, RF_PAGE, hd], value pages [n_pages, nkv, RF_PAGE, hdv].
// What the per-head writer does beyond norm and rotation (all off when zero): a bias on the q | k | v columns, the norm
// taken after the rotation instead of before it, a temperature on the queries, 1 + q_coef ln(floor((pos + 1) / q_every) + 1),
// and rows without value columns whose keys are also their values (q | k; the caller reads values from the key pages).
struct HeadWriteExtras {
    const void* bias;
    int bias_is_f32;
    int norm_after;
    float q_coef;
    float q_every;
    int v_is_k;
};

template <typename T, bool PARTIALS>
__global__ void __launch_bounds__(128)
head_norm_kv_write_kernel(const void* __restrict__ src, int row_stride, int n_partials, size_t partial_stride,
                          T* __restrict__ q_out, int q_out_stride, int nh, int nkv, int hd, int hdv,
                          const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
                          const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                          const int* __restrict__ block_table, int max_pages, T* __restrict__ k_pages,
                          T* __restrict__ v_pages, int write_kv, int rot_dim, int interleaved, int unit_norm, float eps,
                          const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_w_is_f32,
                          float magnitude, HeadWriteExtras ex) {
    extern __shared__ float heads_buf[];            // [warps][2][max(hd, hdv)]
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int hmax = hd > hdv ? hd : hdv;
    float* buf = heads_buf + warp * 2 * hmax;
    float* turned = buf + hmax;
    const int pos = tok_pos[t];
    const int slot = seq_slot[tok_seq[t]];
    const int page = write_kv ? block_table[(size_t)slot * max_pages + pos / RF_PAGE] : 0;
    const int rh = rot_dim >> 1;
    // a query's temperature grows with its position in steps of q_every positions
    const float q_temp = ex.q_every > 0.f ? 1.f + ex.q_coef * logf(floorf((float)(pos + 1) / ex.q_every) + 1.f) : 1.f;
    pdl_wait();
    const int n_heads_all = write_kv ? nh + (ex.v_is_k ? 1 : 2) * nkv : nh;
    for (int head = blockIdx.y * nwarp + warp; head < n_heads_all; head += gridDim.y * nwarp) {
        const bool is_v = head >= nh + nkv;
        const int n = is_v ? hdv : hd;
        const int col = is_v ? (nh + nkv) * hd + (head - nh - nkv) * hdv : head * hd;
        float ss = 0.f;
        for (int e = lane; e < n; e += 32) {
            float x;
            if (PARTIALS) {
                const float* p = reinterpret_cast<const float*>(src) + (size_t)t * row_stride + col + e;
                x = 0.f;
#pragma unroll 4
                for (int sp = 0; sp < n_partials; ++sp) x += p[(size_t)sp * partial_stride];
            } else {
                x = Cvt<T>::to_f32(reinterpret_cast<const T*>(src)[(size_t)t * row_stride + col + e]);
            }
            if (ex.bias != nullptr) x += load_vec(ex.bias, ex.bias_is_f32, col + e);
            buf[e] = x;
            ss += x * x;
        }
        const bool normed = unit_norm && !is_v;
        float r = 1.f;
        if (normed && !ex.norm_after) r = rsqrtf(warp_sum(ss) / (float)n + eps);
        const void* nw = normed ? (head < nh ? q_norm_w : k_norm_w) : nullptr;
        __syncwarp();
        if (nw != nullptr && !ex.norm_after) {            // the weighted norm comes before the rotation
            for (int e = lane; e < n; e += 32) buf[e] *= load_vec(nw, norm_w_is_f32, e);
            __syncwarp();
        }
        T* dst = head < nh ? q_out + (size_t)t * q_out_stride + (size_t)head * hd
               : !is_v ? k_pages + ((size_t)page * nkv + (head - nh)) * RF_PAGE * hd + (size_t)(pos % RF_PAGE) * hd
                       : v_pages + ((size_t)page * nkv + (head - nh - nkv)) * RF_PAGE * hdv + (size_t)(pos % RF_PAGE) * hdv;
        const float out_scale = head < nh ? q_temp : 1.f;
        float ss2 = 0.f;
        for (int e = lane; e < n; e += 32) {
            float x = buf[e] * r;
            if (!is_v && e < rot_dim) {
                int i, partner; bool first;
                if (interleaved) { i = e >> 1; first = !(e & 1); partner = first ? e + 1 : e - 1; }
                else { first = e < rh; i = first ? e : e - rh; partner = first ? e + rh : e - rh; }
                float s, c;
                sincosf((float)pos * inv_freq[i], &s, &c);
                s *= magnitude; c *= magnitude;           // encodings that lengthen the rotated pairs (1: a pure rotation)
                const float y = buf[partner] * r;
                x = first ? x * c - y * s : x * c + y * s;
            }
            if (normed && ex.norm_after) { turned[e] = x; ss2 += x * x; }
            else dst[e] = Cvt<T>::from_f32(x * out_scale);
        }
        if (normed && ex.norm_after) {                    // the head is divided by its root mean square as it is after the rotation
            const float r2 = rsqrtf(warp_sum(ss2) / (float)n + eps);
            for (int e = lane; e < n; e += 32) {          // (a lane reads what it wrote)
                float x = turned[e] * r2;
                if (nw != nullptr) x *= load_vec(nw, norm_w_is_f32, e);
                dst[e] = Cvt<T>::from_f32(x * out_scale);
            }
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------- gated unit with clamped halves
// a[t, j] = g sigmoid(alpha g) (u + 1) with g = min(gu[t, 2j], limit), u = clamp(gu[t, 2j+1], -limit, limit), evaluated in
// 32-bit.  row_scale (float [T], may be null) multiplies both halves of row t first: W (s x) = s (W x), so an input that
// is scaled by a routing score can be given as the unscaled product and the score.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ a, size_t n_out, int I, float limit, float alpha,
                                   const float* __restrict__ row_scale) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_out; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, j = idx - t * I;
        const float sc = row_scale != nullptr ? row_scale[t] : 1.f;
        const float g = fminf(Cvt<T>::to_f32(gu[t * 2 * I + 2 * j]) * sc, limit);
        const float u = fminf(fmaxf(Cvt<T>::to_f32(gu[t * 2 * I + 2 * j + 1]) * sc, -limit), limit);
        a[idx] = Cvt<T>::from_f32(g / (1.f + expf(-alpha * g)) * (u + 1.f));
    }
}

// ---------------------------------------------------------------- out[t, c] = x[t, c] * sigmoid(gate[t, c / group])
// group 1: a gate per element; group = a head's size: one gate per head
template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ gate, int gate_stride,
                                    T* __restrict__ out, size_t n, int W, int group) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / W, c = idx - t * W;
        const float g = Cvt<T>::to_f32(gate[t * gate_stride + c / group]);
        out[idx] = Cvt<T>::from_f32(Cvt<T>::to_f32(x[t * x_stride + c]) / (1.f + expf(-g)));
    }
}

// The same, 16 bytes of a row a thread (W, the rows' strides and, with a gate per element, the gates' stride are whole
// numbers of such groups; with a gate per head a group lies inside one head).  Every element is formed as above.
template <typename T, bool PER_ELEMENT>
__global__ void sigmoid_gate_vec_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ gate, int gate_stride,
                                        T* __restrict__ out, size_t n_vec, int Wv, int group) {
    constexpr int V = 16 / sizeof(T);
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n_vec; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / Wv;
        const int c = (int)(idx - t * Wv) * V;
        alignas(16) T xs[V], gs[V], ys[V];
        *reinterpret_cast<uint4*>(xs) = *reinterpret_cast<const uint4*>(x + t * x_stride + c);
        if (PER_ELEMENT) {
            *reinterpret_cast<uint4*>(gs) = *reinterpret_cast<const uint4*>(gate + t * gate_stride + c);
#pragma unroll
            for (int u = 0; u < V; ++u)
                ys[u] = Cvt<T>::from_f32(Cvt<T>::to_f32(xs[u]) / (1.f + expf(-Cvt<T>::to_f32(gs[u]))));
        } else {
            const float d = 1.f + expf(-Cvt<T>::to_f32(gate[t * gate_stride + c / group]));
#pragma unroll
            for (int u = 0; u < V; ++u) ys[u] = Cvt<T>::from_f32(Cvt<T>::to_f32(xs[u]) / d);
        }
        *reinterpret_cast<uint4*>(out + t * (size_t)(Wv * V) + c) = *reinterpret_cast<const uint4*>(ys);
    }
}

// ---------------------------------------------------------------- the 32-bit stream rounded to the compute dtype
template <typename T>
__global__ void round_rows_kernel(const float* __restrict__ h, T* __restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = Cvt<T>::from_f32(h[idx]);
}

// ---------------------------------------------------------------- Dynamic Tanh: a norm without statistics
// y = tanh(alpha h) * w + b, element by element (alpha one number), of the rows that `rows` lists (null: all).  The
// vectors and alpha are 32-bit.
template <typename T>
__global__ void dyt_rows_kernel(const float* __restrict__ h, const int* __restrict__ rows, const float* __restrict__ alpha,
                                const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ y, int H) {
    pdl_trigger();
    const float a = alpha[0];
    pdl_wait();
    const size_t src = (size_t)(rows != nullptr ? rows[blockIdx.x] : (int)blockIdx.x) * H, dst = (size_t)blockIdx.x * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) y[dst + c] = Cvt<T>::from_f32(fmaf(tanhf(a * h[src + c]), w[c], b[c]));
}

// ---------------------------------------------------------------- a scaled update of the stream
// The residual update of a block that scales its sub-layers' outputs, all in 32-bit:
//   m = a0 (+ a1)                                     (one result, or two that are summed: w0 null), or
//   m = (rms(a0) * w0 + rms(a1) * w1) / 2             (two branches side by side, each normed with its own weight)
//   h += mult * m
//   y_next = tanh(alpha h) * w_next + b_next          in the compute dtype, if the caller knows the norm that reads the
//                                                      stream next (a Dynamic Tanh)
// with rms(x) = x / sqrt(mean(x^2) + eps).  a0 (a1) comes as n0 (n1) partial sums [n][rows][H] of a K-split product,
// added here in index order.  A block per row.
template <typename T>
__global__ void __launch_bounds__(1024)
scaled_add_kernel(float* __restrict__ h, const float* __restrict__ a0, int n0, const void* __restrict__ w0,
                  const float* __restrict__ a1, int n1, size_t part_stride, const void* __restrict__ w1, int w_is_f32,
                  float eps, float mult, const float* __restrict__ alpha, const float* __restrict__ w_next,
                  const float* __restrict__ b_next, T* __restrict__ y_next, int H) {
    extern __shared__ float row[];                  // [H], a second [H] for the other branch, 34 for the sums
    float* other = row + H;
    float* red = other + H;
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * H;
    const float invH = 1.f / (float)H;
    const float a = y_next != nullptr ? alpha[0] : 0.f;
    pdl_wait();
    float s0 = 0.f, s1 = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x = 0.f, z = 0.f;
#pragma unroll 4
        for (int s = 0; s < n0; ++s) x += a0[(size_t)s * part_stride + base + c];
        if (a1 != nullptr) {
#pragma unroll 4
            for (int s = 0; s < n1; ++s) z += a1[(size_t)s * part_stride + base + c];
        }
        row[c] = x; other[c] = z;
        s0 += x * x; s1 += z * z;
    }
    float r0 = 1.f, r1 = 1.f;
    if (w0 != nullptr) {
        r0 = rsqrtf(block_sum(s0, red) * invH + eps);
        r1 = rsqrtf(block_sum(s1, red) * invH + eps);
    }
    for (int c = threadIdx.x; c < H; c += blockDim.x) {      // a thread reads what it wrote
        const float m = w0 != nullptr
            ? 0.5f * (row[c] * r0 * load_vec(w0, w_is_f32, c) + other[c] * r1 * load_vec(w1, w_is_f32, c))
            : row[c] + other[c];
        const float v = fmaf(mult, m, h[base + c]);
        h[base + c] = v;
        if (y_next != nullptr) y_next[base + c] = Cvt<T>::from_f32(fmaf(tanhf(a * v), w_next[c], b_next[c]));
    }
}

// ---------------------------------------------------------------- h += s0 * a0 + s1 * a1, then the next RMS norm
// Two sub-layer results side by side, each float32 [rows][H] or a stack of n partial sums added in index order, each
// with a factor of its own; the sum goes into the 32-bit stream.  With w_next the norm that reads the stream next is
// computed in the same pass: y = h / sqrt(mean(h^2) + eps) * w_next, in the compute dtype.
template <typename T>
__global__ void __launch_bounds__(1024)
weighted_add_kernel(float* __restrict__ h, const float* __restrict__ a0, int n0, float s0, const float* __restrict__ a1, int n1,
                    float s1, size_t part_stride, const void* __restrict__ w_next, int w_is_f32, float eps,
                    T* __restrict__ y_next, int H) {
    extern __shared__ float row[];                  // [H], 34 for the sums
    float* red = row + H;
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * H;
    pdl_wait();
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x = 0.f, z = 0.f;
#pragma unroll 4
        for (int s = 0; s < n0; ++s) x += a0[(size_t)s * part_stride + base + c];
        if (a1 != nullptr) {
#pragma unroll 4
            for (int s = 0; s < n1; ++s) z += a1[(size_t)s * part_stride + base + c];
        }
        const float v = h[base + c] + (s0 * x + s1 * z);
        h[base + c] = v;
        row[c] = v;
        ss += v * v;
    }
    if (y_next == nullptr) return;
    const float r = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)        // a thread reads what it wrote
        y_next[base + c] = Cvt<T>::from_f32(row[c] * r * load_vec(w_next, w_is_f32, c));
}

template <typename T>
static int launch_weighted_add(float* h, const float* a0, int n0, float s0, const float* a1, int n1, float s1,
                               const void* w_next, int w_is_f32, float eps, void* y_next, int rows, int H, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (a0 == nullptr || n0 < 1 || (a1 != nullptr && n1 < 1) || (y_next != nullptr && w_next == nullptr)) return RF_ERR_BAD_ARG;
    const size_t smem = ((size_t)H + 34) * sizeof(float);
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(weighted_add_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    int threads = 256;
    if (rows <= 296) { threads = (H + 31) / 32 * 32; if (threads > 1024) threads = 1024; if (threads < 256) threads = 256; }
    rf_launch(weighted_add_kernel<T>, dim3(rows), dim3(threads), smem, st, h, a0, n0, s0, a1, n1, s1, (size_t)rows * H, w_next,
              w_is_f32, eps, reinterpret_cast<T*>(y_next), H);
    RF_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- RMS norms of stretches of a row
// Block (t, j) norms columns col[j] .. col[j] + n[j] of row t of src: y = x / sqrt(mean(x^2) + eps) * w_j (w_j null: no
// weight), sums in 32-bit, and writes them to out_j [T][n_j] (row stride given).  Up to two stretches a launch.
struct NormStretch {
    int col, n;
    const void* w;
    void* out;
    int out_stride;
};
template <typename T>
__global__ void __launch_bounds__(256)
stretch_norm_kernel(const T* __restrict__ src, int src_stride, NormStretch a, NormStretch b, int w_is_f32, float eps) {
    __shared__ float red[34];
    pdl_trigger();
    const NormStretch s = blockIdx.y == 0 ? a : b;
    const T* x = src + (size_t)blockIdx.x * src_stride + s.col;
    T* y = reinterpret_cast<T*>(s.out) + (size_t)blockIdx.x * s.out_stride;
    pdl_wait();
    float ss = 0.f;
    for (int c = threadIdx.x; c < s.n; c += blockDim.x) { const float v = Cvt<T>::to_f32(x[c]); ss += v * v; }
    const float r = rsqrtf(block_sum(ss, red) / (float)s.n + eps);
    for (int c = threadIdx.x; c < s.n; c += blockDim.x)
        y[c] = Cvt<T>::from_f32(Cvt<T>::to_f32(x[c]) * r * (s.w != nullptr ? load_vec(s.w, w_is_f32, c) : 1.f));
}

// ---------------------------------------------------------------- x <- cap * tanh(x / cap), in place (logits)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_trigger();
    pdl_wait();
    const float inv = 1.f / cap;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x)
        x[idx] = cap * tanhf(x[idx] * inv);
}

template <typename T>
static int launch_dyt_rows(const float* h, const int* rows, const float* alpha, const float* w, const float* b, void* y, int R,
                           int H, cudaStream_t st) {
    if (R <= 0) return 0;
    int threads = (H + 3) / 4;
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : (threads + 31) / 32 * 32);
    rf_launch(dyt_rows_kernel<T>, dim3(R), dim3(threads), 0, st, h, rows, alpha, w, b, reinterpret_cast<T*>(y), H);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_scaled_add(float* h, const float* a0, int n0, const void* w0, const float* a1, int n1, const void* w1,
                             int w_is_f32, float eps, float mult, const float* alpha, const float* w_next,
                             const float* b_next, void* y_next, int rows, int H, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (n0 < 1 || (a1 != nullptr && n1 < 1) || (w0 != nullptr && (a1 == nullptr || w1 == nullptr))) return RF_ERR_BAD_ARG;
    if (y_next != nullptr && (alpha == nullptr || w_next == nullptr || b_next == nullptr)) return RF_ERR_BAD_ARG;
    const size_t smem = (size_t)(2 * H + 34) * sizeof(float);
    if (smem > 200 * 1024) return RF_ERR_UNSUPPORTED;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(scaled_add_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    int threads = 256;
    if (rows <= 296) { threads = (H + 31) / 32 * 32; if (threads > 1024) threads = 1024; if (threads < 256) threads = 256; }
    rf_launch(scaled_add_kernel<T>, dim3(rows), dim3(threads), smem, st, h, a0, n0, w0, a1, n1, (size_t)rows * H, w1, w_is_f32,
              eps, mult, alpha, w_next, b_next, reinterpret_cast<T*>(y_next), H);
    RF_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- launchers
template <typename T>
static int launch_clamped_glu(const void* gu, void* a, int T_, int I, float limit, float alpha, const float* row_scale,
                              cudaStream_t st) {
    const size_t n = (size_t)T_ * I;
    if (n == 0) return 0;
    const size_t blocks = (n + 255) / 256;
    rf_launch(clamped_glu_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st,
              reinterpret_cast<const T*>(gu), reinterpret_cast<T*>(a), n, I, limit, alpha, row_scale);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_sigmoid_gate(const void* x, int x_stride, const void* gate, int gate_stride, void* out, int T_, int W,
                               int group, cudaStream_t st) {
    if (group < 1) return RF_ERR_BAD_ARG;
    const size_t n = (size_t)T_ * W;
    if (n == 0) return 0;
    constexpr int V = 16 / (int)sizeof(T);
    auto whole = [](const void* p, int stride) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && stride % V == 0; };
    if (W % V == 0 && whole(x, x_stride) && whole(out, W) && (group == 1 ? whole(gate, gate_stride) : group % V == 0)) {
        const size_t n_vec = n / V, vblocks = (n_vec + 255) / 256;
        const dim3 grid((unsigned)(vblocks > 148 * 16 ? 148 * 16 : vblocks));
        if (group == 1)
            rf_launch(sigmoid_gate_vec_kernel<T, true>, grid, dim3(256), 0, st, reinterpret_cast<const T*>(x), x_stride,
                      reinterpret_cast<const T*>(gate), gate_stride, reinterpret_cast<T*>(out), n_vec, W / V, group);
        else
            rf_launch(sigmoid_gate_vec_kernel<T, false>, grid, dim3(256), 0, st, reinterpret_cast<const T*>(x), x_stride,
                      reinterpret_cast<const T*>(gate), gate_stride, reinterpret_cast<T*>(out), n_vec, W / V, group);
        RF_LAUNCH_CHECK();
        return 0;
    }
    const size_t blocks = (n + 255) / 256;
    rf_launch(sigmoid_gate_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st,
              reinterpret_cast<const T*>(x), x_stride, reinterpret_cast<const T*>(gate), gate_stride, reinterpret_cast<T*>(out), n, W, group);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_round_rows(const float* h, void* out, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    rf_launch(round_rows_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st, h,
              reinterpret_cast<T*>(out), (size_t)n);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_embed(const void* table, const int* ids, float* out, int T_, int H, int V, cudaStream_t st,
                        const void* pos_table = nullptr, const int* tok_pos = nullptr, int P = 0, void* rounded = nullptr,
                        float scale = 1.f) {
    if (T_ <= 0) return 0;
    if (pos_table != nullptr && (tok_pos == nullptr || P <= 0)) return RF_ERR_BAD_ARG;
    rf_launch(embed_kernel<T>, dim3(T_), dim3(256), 0, st, reinterpret_cast<const T*>(table), ids, out, H, V,
              reinterpret_cast<const T*>(pos_table), tok_pos, P, reinterpret_cast<T*>(rounded), scale);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_add_rmsnorm(float* h, const void* pending, int kind, int n_pending, size_t pstride,
                              const void* w, int w_is_f32, float eps, void* y, const int* rows,
                              int n_rows, int H, int* status, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (H % 4 == 0 && H <= 4 * 4 * 1024 && (pstride % 4) == 0 &&
        !(reinterpret_cast<uintptr_t>(h) & 15) && !(reinterpret_cast<uintptr_t>(w) & 15) && !(reinterpret_cast<uintptr_t>(y) & 15) &&
        !(kind == 1 && (reinterpret_cast<uintptr_t>(pending) & 15))) {
        const int nvec = H / 4;
        if (kind == 0 && !rows && n_rows >= 512) {       // a prompt step's norm: rows read twice, eight CTAs per SM
            rf_launch(rmsnorm_rows_kernel<T>, dim3(n_rows), dim3(256), 0, st, (const float*)h, w, w_is_f32, eps, reinterpret_cast<T*>(y), H);
            RF_LAUNCH_CHECK();
            return 0;
        }
        // few rows (decode): one 16-byte vector per thread, the shortest chain per row;
        // many rows (prompts): 256 threads a row, so that eight rows per SM are in flight
        int threads = ((nvec + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (n_rows >= 512 && nvec > 256 && nvec <= 1024) threads = 256;
        const int per = (nvec + threads - 1) / threads;
        T* yy = reinterpret_cast<T*>(y);
        // few rows: the row's threads as a cluster of up to 8 CTAs of whole warps, while that makes no more CTAs than
        // two per SM
        int cl = 1;
        for (int c = 8; c >= 2; --c)
            if ((threads / 32) % c == 0 && (long long)n_rows * c <= 296) { cl = c; break; }
        const dim3 grid(n_rows * cl), block(threads / cl);
        auto go = [&](auto kernel) {
            if (cl > 1) rf_launch_cluster(kernel, grid, block, 0, st, cl, h, pending, kind, n_pending, pstride, w, w_is_f32, eps, yy, rows, H, cl, status);
            else rf_launch(kernel, grid, block, 0, st, h, pending, kind, n_pending, pstride, w, w_is_f32, eps, yy, rows, H, cl, status);
        };
        const bool wide = block.x <= 256 && kind == 1 && n_pending > 4;      // K splits to add up, and room for the registers
        if (per <= 1 && wide) go(add_rmsnorm_vec_kernel<T, 1, 16, 256>);
        else if (per <= 2 && wide) go(add_rmsnorm_vec_kernel<T, 2, 8, 256>);
        else if (per <= 1) go(add_rmsnorm_vec_kernel<T, 1, 4, 1024>);
        else if (per <= 2) go(add_rmsnorm_vec_kernel<T, 2, 4, 1024>);
        else go(add_rmsnorm_vec_kernel<T, 4, 4, 1024>);
        RF_LAUNCH_CHECK();
        return 0;
    }
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return RF_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = H >= 2048 ? 512 : 256;
    rf_launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, st, h, pending, kind, n_pending, pstride, w,
              w_is_f32, eps, reinterpret_cast<T*>(y), rows, H);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_rope_kv_write(const void* src, int row_stride, int n_partials, size_t partial_stride,
                                const void* bias, int bias_is_f32, void* q_out, int q_out_stride, int nh, int nkv,
                                int hd, const float* inv_freq, const int* tok_seq, const int* tok_pos,
                                const int* seq_slot, const int* block_table, int max_pages, void* k_pages,
                                void* v_pages, int write_kv, int T_, int rot_dim, int interleaved, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (hd % 2 || rot_dim % 2 || rot_dim < 0 || rot_dim > hd) return RF_ERR_BAD_ARG;
    const int n_pairs = (nh + 2 * nkv) * (hd / 2);
    const dim3 grid(T_, (n_pairs + 255) / 256);
    if (T_ > 2147483647 || grid.y > 65535) return RF_ERR_UNSUPPORTED;
    // prompts: rows of one tensor, everything aligned for accesses of four elements
    const size_t four = 4 * sizeof(T);
    auto aligned = [&](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) % four) == 0; };
    if (n_partials == 0 && rot_dim == hd && !interleaved && T_ >= 64 && hd % 8 == 0 && hd / 8 <= 256 && row_stride % 4 == 0 && q_out_stride % 4 == 0 &&
        aligned(src) && aligned(q_out) && (!write_kv || (aligned(k_pages) && aligned(v_pages)))) {
        const int groups = hd / 8;
        int threads = ((nh + 2 * nkv) * groups + 31) / 32 * 32;        // a row of groups per head, at most 256 threads
        if (threads > 256) threads = 256;
        if (threads < groups) threads = (groups + 31) / 32 * 32;
        rf_launch(rope_kv_write_rows_kernel<T>, dim3(T_), dim3(threads), 0, st, reinterpret_cast<const T*>(src), row_stride,
            reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
            max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv);
        RF_LAUNCH_CHECK();
        return 0;
    }
    if (n_partials > 0)
        rf_launch(rope_kv_write_kernel<T, true>, grid, dim3(256), 0, st, src, row_stride, n_partials, partial_stride, bias,
            bias_is_f32, reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot,
            block_table, max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv, rot_dim,
            interleaved);
    else
        rf_launch(rope_kv_write_kernel<T, false>, grid, dim3(256), 0, st, src, row_stride, 0, (size_t)0, (const void*)nullptr, 0,
            reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot,
            block_table, max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv, rot_dim,
            interleaved);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_swiglu(const void* gu, void* a, int T_, int I, cudaStream_t st) {
    const size_t n = (size_t)T_ * I;
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    rf_launch(swiglu_kernel<T>, dim3(blocks), dim3(256), 0, st, reinterpret_cast<const T*>(gu), reinterpret_cast<T*>(a), n, I);
    RF_LAUNCH_CHECK();
    return 0;
}


template <typename T>
static int launch_relu2(const void* x, void* a, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    rf_launch(relu2_kernel<T>, dim3(blocks), dim3(256), 0, st, reinterpret_cast<const T*>(x), reinterpret_cast<T*>(a), (size_t)n);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_add_row(float* h, const void* vec, int T_, int H, cudaStream_t st) {
    const size_t n = (size_t)T_ * H;
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    rf_launch(add_row_kernel<T>, dim3(blocks), dim3(256), 0, st, h, reinterpret_cast<const T*>(vec), n, H);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_branch_norm_add(float* h, const float* a0, int n0, const void* w0, const float* a1, int n1,
                                  const void* w1, const void* w_post, const void* extra, const void* w_next, void* y_next,
                                  int w_is_f32, float eps, int rows, int H, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (n0 < 1 || (a1 != nullptr && n1 < 1)) return RF_ERR_BAD_ARG;
    const size_t smem = (size_t)(2 * H + 34) * sizeof(float);
    if (smem > 200 * 1024) return RF_ERR_UNSUPPORTED;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(branch_norm_add_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    // few rows (decode): a row's columns over up to 1024 threads, so that its loads are all in flight at once
    int threads = 256;
    if (rows <= 296) { threads = (H + 31) / 32 * 32; if (threads > 1024) threads = 1024; if (threads < 256) threads = 256; }
    rf_launch(branch_norm_add_kernel<T>, dim3(rows), dim3(threads), smem, st, h, a0, n0, w0, a1, n1, (size_t)rows * H, w1, w_post,
              extra, w_next, reinterpret_cast<T*>(y_next), w_is_f32, eps, H);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_head_norm_kv_write(const void* src, int row_stride, int n_partials, size_t partial_stride, void* q_out,
                                     int q_out_stride, int nh, int nkv, int hd, int hdv, const float* inv_freq,
                                     const int* tok_seq, const int* tok_pos, const int* seq_slot, const int* block_table,
                                     int max_pages, void* k_pages, void* v_pages, int write_kv, int T_, int rot_dim,
                                     int interleaved, int unit_norm, float eps, cudaStream_t st,
                                     const void* q_norm_w = nullptr, const void* k_norm_w = nullptr, int norm_w_is_f32 = 0,
                                     float magnitude = 1.f, HeadWriteExtras ex = HeadWriteExtras{nullptr, 0, 0, 0.f, 0.f, 0}) {
    if (T_ <= 0) return 0;
    if (rot_dim % 2 || rot_dim < 0 || rot_dim > hd || hd <= 0 || hdv <= 0 || ex.q_every < 0.f) return RF_ERR_BAD_ARG;
    const size_t smem = (size_t)4 * 2 * (hd > hdv ? hd : hdv) * sizeof(float);
    if (smem > 48 * 1024) return RF_ERR_UNSUPPORTED;
    // few tokens: a token's heads over several blocks (a warp per head)
    const int all_heads = write_kv ? nh + (ex.v_is_k ? 1 : 2) * nkv : nh;
    int by = T_ >= 512 ? 1 : (all_heads + 3) / 4;
    if (by > 64) by = 64;
    if (n_partials > 0)
        rf_launch(head_norm_kv_write_kernel<T, true>, dim3(T_, by), dim3(128), smem, st, src, row_stride, n_partials, partial_stride,
                  reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                  max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv, rot_dim, interleaved, unit_norm, eps,
                  q_norm_w, k_norm_w, norm_w_is_f32, magnitude, ex);
    else
        rf_launch(head_norm_kv_write_kernel<T, false>, dim3(T_, by), dim3(128), smem, st, src, row_stride, 0, (size_t)0,
                  reinterpret_cast<T*>(q_out), q_out_stride, nh, nkv, hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                  max_pages, reinterpret_cast<T*>(k_pages), reinterpret_cast<T*>(v_pages), write_kv, rot_dim, interleaved, unit_norm, eps,
                  q_norm_w, k_norm_w, norm_w_is_f32, magnitude, ex);
    RF_LAUNCH_CHECK();
    return 0;
}

// dtype: 0 = float32, 1 = bfloat16
extern "C" {
int rf_embed(int dtype, const void* table, const int* ids, float* out, int T_, int H, int V, cudaStream_t st) {
    return dtype == 0 ? launch_embed<float>(table, ids, out, T_, H, V, st)
                      : launch_embed<__nv_bfloat16>(table, ids, out, T_, H, V, st);
}
// out[t] = table[ids[t]] * scale, the product formed in 32-bit.
int rf_embed_scaled(int dtype, const void* table, const int* ids, float* out, int T_, int H, int V, float scale, cudaStream_t st) {
    return dtype == 0 ? launch_embed<float>(table, ids, out, T_, H, V, st, nullptr, nullptr, 0, nullptr, scale)
                      : launch_embed<__nv_bfloat16>(table, ids, out, T_, H, V, st, nullptr, nullptr, 0, nullptr, scale);
}
// The same with a learned position table [P, H] (row tok_pos[t] is added; null: none) and a copy of the result in the
// table's dtype (rounded; null: none).
int rf_embed_pos(int dtype, const void* table, const int* ids, float* out, int T_, int H, int V, const void* pos_table,
                 const int* tok_pos, int P, void* rounded, cudaStream_t st) {
    return dtype == 0 ? launch_embed<float>(table, ids, out, T_, H, V, st, pos_table, tok_pos, P, rounded)
                      : launch_embed<__nv_bfloat16>(table, ids, out, T_, H, V, st, pos_table, tok_pos, P, rounded);
}
int rf_add_rmsnorm(int dtype, float* h, const void* pending, int kind, int n_pending, long long pstride,
                   const void* w, int w_is_f32, float eps, void* y, const int* rows, int n_rows, int H,
                   int* status, cudaStream_t st) {
    // status: the device word that a cluster's bounded wait sets to 7 when it runs out (may be null)
    return dtype == 0
        ? launch_add_rmsnorm<float>(h, pending, kind, n_pending, (size_t)pstride, w, w_is_f32, eps, y, rows, n_rows, H, status, st)
        : launch_add_rmsnorm<__nv_bfloat16>(h, pending, kind, n_pending, (size_t)pstride, w, w_is_f32, eps, y, rows, n_rows, H, status, st);
}
int rf_rope_kv_write(int dtype, const void* src, int row_stride, int n_partials, long long partial_stride,
                     const void* bias, int bias_is_f32, void* q_out, int q_out_stride, int nh, int nkv, int hd,
                     const float* inv_freq, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                     const int* block_table, int max_pages, void* k_pages, void* v_pages, int write_kv, int T_,
                     int rot_dim, int interleaved, cudaStream_t st) {
    return dtype == 0
        ? launch_rope_kv_write<float>(src, row_stride, n_partials, (size_t)partial_stride, bias, bias_is_f32, q_out,
                                      q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                                      max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved, st)
        : launch_rope_kv_write<__nv_bfloat16>(src, row_stride, n_partials, (size_t)partial_stride, bias, bias_is_f32,
                                              q_out, q_out_stride, nh, nkv, hd, inv_freq, tok_seq, tok_pos, seq_slot,
                                              block_table, max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved, st);
}
int rf_swiglu(int dtype, const void* gu, void* a, int T_, int I, cudaStream_t st) {
    return dtype == 0 ? launch_swiglu<float>(gu, a, T_, I, st) : launch_swiglu<__nv_bfloat16>(gu, a, T_, I, st);
}
int rf_relu2(int dtype, const void* x, void* a, long long n, cudaStream_t st) {
    return dtype == 0 ? launch_relu2<float>(x, a, n, st) : launch_relu2<__nv_bfloat16>(x, a, n, st);
}
int rf_add_row(int dtype, float* h, const void* vec, int T_, int H, cudaStream_t st) {
    return dtype == 0 ? launch_add_row<float>(h, vec, T_, H, st) : launch_add_row<__nv_bfloat16>(h, vec, T_, H, st);
}
// a1 / w1 null: one branch, taken as it is; extra, w_next / y_next null: left out.  All weight vectors share w_is_f32.
// a0 / a1 are stacks of n0 / n1 partial sums, each [rows][H] (1: the branch itself).
int rf_branch_norm_add(int dtype, float* h, const float* a0, int n0, const void* w0, const float* a1, int n1, const void* w1,
                       const void* w_post, const void* extra, const void* w_next, void* y_next, int w_is_f32, float eps,
                       int rows, int H, cudaStream_t st) {
    return dtype == 0
        ? launch_branch_norm_add<float>(h, a0, n0, w0, a1, n1, w1, w_post, extra, w_next, y_next, w_is_f32, eps, rows, H, st)
        : launch_branch_norm_add<__nv_bfloat16>(h, a0, n0, w0, a1, n1, w1, w_post, extra, w_next, y_next, w_is_f32, eps, rows, H, st);
}
int rf_head_norm_kv_write(int dtype, const void* src, int row_stride, int n_partials, long long partial_stride, void* q_out,
                          int q_out_stride, int nh, int nkv, int hd, int hdv, const float* inv_freq, const int* tok_seq,
                          const int* tok_pos, const int* seq_slot, const int* block_table, int max_pages, void* k_pages,
                          void* v_pages, int write_kv, int T_, int rot_dim, int interleaved, int unit_norm, float eps,
                          cudaStream_t st) {
    return dtype == 0
        ? launch_head_norm_kv_write<float>(src, row_stride, n_partials, (size_t)partial_stride, q_out, q_out_stride, nh, nkv,
                                           hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table, max_pages, k_pages,
                                           v_pages, write_kv, T_, rot_dim, interleaved, unit_norm, eps, st)
        : launch_head_norm_kv_write<__nv_bfloat16>(src, row_stride, n_partials, (size_t)partial_stride, q_out, q_out_stride,
                                                   nh, nkv, hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                                                   max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved,
                                                   unit_norm, eps, st);
}
// The same with weights of the q and k norms (each [hd], shared by the heads; null: a plain division) and a factor on the
// rotation's sine and cosine (1: a pure rotation).
int rf_head_norm_kv_write_w(int dtype, const void* src, int row_stride, int n_partials, long long partial_stride, void* q_out,
                            int q_out_stride, int nh, int nkv, int hd, int hdv, const float* inv_freq, const int* tok_seq,
                            const int* tok_pos, const int* seq_slot, const int* block_table, int max_pages, void* k_pages,
                            void* v_pages, int write_kv, int T_, int rot_dim, int interleaved, int unit_norm, float eps,
                            const void* q_norm_w, const void* k_norm_w, int norm_w_is_f32, float magnitude, cudaStream_t st) {
    return dtype == 0
        ? launch_head_norm_kv_write<float>(src, row_stride, n_partials, (size_t)partial_stride, q_out, q_out_stride, nh, nkv,
                                           hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table, max_pages, k_pages,
                                           v_pages, write_kv, T_, rot_dim, interleaved, unit_norm, eps, st, q_norm_w, k_norm_w,
                                           norm_w_is_f32, magnitude)
        : launch_head_norm_kv_write<__nv_bfloat16>(src, row_stride, n_partials, (size_t)partial_stride, q_out, q_out_stride,
                                                   nh, nkv, hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                                                   max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved,
                                                   unit_norm, eps, st, q_norm_w, k_norm_w, norm_w_is_f32, magnitude);
}
// The same with a bias on the columns read ([q | k | v], null: none), the norm taken after the rotation (norm_after), a
// temperature on the queries (q_every > 0: 1 + q_coef ln(floor((pos + 1) / q_every) + 1)) and rows q | k whose keys are
// their values (v_is_k: nothing is written to value pages).
int rf_head_norm_kv_write_x(int dtype, const void* src, int row_stride, int n_partials, long long partial_stride, void* q_out,
                            int q_out_stride, int nh, int nkv, int hd, int hdv, const float* inv_freq, const int* tok_seq,
                            const int* tok_pos, const int* seq_slot, const int* block_table, int max_pages, void* k_pages,
                            void* v_pages, int write_kv, int T_, int rot_dim, int interleaved, int unit_norm, float eps,
                            const void* q_norm_w, const void* k_norm_w, int norm_w_is_f32, float magnitude,
                            const void* bias, int bias_is_f32, int norm_after, float q_coef, float q_every, int v_is_k,
                            cudaStream_t st) {
    const HeadWriteExtras ex{bias, bias_is_f32, norm_after, q_coef, q_every, v_is_k};
    return dtype == 0
        ? launch_head_norm_kv_write<float>(src, row_stride, n_partials, (size_t)partial_stride, q_out, q_out_stride, nh, nkv,
                                           hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table, max_pages, k_pages,
                                           v_pages, write_kv, T_, rot_dim, interleaved, unit_norm, eps, st, q_norm_w, k_norm_w,
                                           norm_w_is_f32, magnitude, ex)
        : launch_head_norm_kv_write<__nv_bfloat16>(src, row_stride, n_partials, (size_t)partial_stride, q_out, q_out_stride,
                                                   nh, nkv, hd, hdv, inv_freq, tok_seq, tok_pos, seq_slot, block_table,
                                                   max_pages, k_pages, v_pages, write_kv, T_, rot_dim, interleaved,
                                                   unit_norm, eps, st, q_norm_w, k_norm_w, norm_w_is_f32, magnitude, ex);
}
int rf_clamped_glu(int dtype, const void* gu, void* a, int T_, int I, float limit, float alpha, const float* row_scale,
                   cudaStream_t st) {
    return dtype == 0 ? launch_clamped_glu<float>(gu, a, T_, I, limit, alpha, row_scale, st)
                      : launch_clamped_glu<__nv_bfloat16>(gu, a, T_, I, limit, alpha, row_scale, st);
}
int rf_sigmoid_gate(int dtype, const void* x, int x_stride, const void* gate, int gate_stride, void* out, int T_, int W,
                    int group, cudaStream_t st) {
    return dtype == 0 ? launch_sigmoid_gate<float>(x, x_stride, gate, gate_stride, out, T_, W, group, st)
                      : launch_sigmoid_gate<__nv_bfloat16>(x, x_stride, gate, gate_stride, out, T_, W, group, st);
}
int rf_round_rows(int dtype, const float* h, void* out, long long n, cudaStream_t st) {
    return dtype == 0 ? launch_round_rows<float>(h, out, n, st) : launch_round_rows<__nv_bfloat16>(h, out, n, st);
}
// y [R, H] of dtype = tanh(alpha h[rows]) * w + b; rows null: every row of h [R, H]
int rf_dyt_rows(int dtype, const float* h, const int* rows, const float* alpha, const float* w, const float* b, void* y,
                int R, int H, cudaStream_t st) {
    return dtype == 0 ? launch_dyt_rows<float>(h, rows, alpha, w, b, y, R, H, st)
                      : launch_dyt_rows<__nv_bfloat16>(h, rows, alpha, w, b, y, R, H, st);
}
// w0 / w1 null: h += mult * (a0 + a1) (a1 null: a0 alone); else h += mult * mean of the two normed branches.  y_next
// (of dtype) null: no next norm.  w0, w1 share w_is_f32; alpha, w_next, b_next are float.
int rf_scaled_add(int dtype, float* h, const float* a0, int n0, const void* w0, const float* a1, int n1, const void* w1,
                  int w_is_f32, float eps, float mult, const float* alpha, const float* w_next, const float* b_next,
                  void* y_next, int rows, int H, cudaStream_t st) {
    return dtype == 0
        ? launch_scaled_add<float>(h, a0, n0, w0, a1, n1, w1, w_is_f32, eps, mult, alpha, w_next, b_next, y_next, rows, H, st)
        : launch_scaled_add<__nv_bfloat16>(h, a0, n0, w0, a1, n1, w1, w_is_f32, eps, mult, alpha, w_next, b_next, y_next, rows, H, st);
}
// h [rows][H] += s0 * sum(a0 parts) + s1 * sum(a1 parts) (a1 null: one addend); with y_next (of dtype) also the RMS norm of
// the new rows with w_next and eps.
int rf_weighted_add(int dtype, float* h, const float* a0, int n0, float s0, const float* a1, int n1, float s1,
                    const void* w_next, int w_is_f32, float eps, void* y_next, int rows, int H, cudaStream_t st) {
    return dtype == 0 ? launch_weighted_add<float>(h, a0, n0, s0, a1, n1, s1, w_next, w_is_f32, eps, y_next, rows, H, st)
                      : launch_weighted_add<__nv_bfloat16>(h, a0, n0, s0, a1, n1, s1, w_next, w_is_f32, eps, y_next, rows, H, st);
}
// RMS norms of one or two stretches of the rows of src [T][src_stride] (n1 0: one stretch); see stretch_norm_kernel.
int rf_stretch_norm(int dtype, const void* src, int src_stride, int col0, int n0, const void* w0, void* out0, int out0_stride,
                    int col1, int n1, const void* w1, void* out1, int out1_stride, int w_is_f32, float eps, int T_,
                    cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (n0 <= 0 || n1 < 0) return RF_ERR_BAD_ARG;
    const NormStretch a{col0, n0, w0, out0, out0_stride}, b{col1, n1, w1, out1, out1_stride};
    const dim3 grid(T_, n1 > 0 ? 2 : 1);
    if (dtype == 0) rf_launch(stretch_norm_kernel<float>, grid, dim3(256), 0, st, reinterpret_cast<const float*>(src), src_stride, a, b, w_is_f32, eps);
    else rf_launch(stretch_norm_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(src), src_stride, a, b, w_is_f32, eps);
    RF_LAUNCH_CHECK();
    return 0;
}
int rf_softcap(float* x, long long n, float cap, cudaStream_t st) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return RF_ERR_BAD_ARG;
    const long long blocks = (n + 255) / 256;
    rf_launch(softcap_kernel, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st, x, (size_t)n, cap);
    RF_LAUNCH_CHECK();
    return 0;
}
}
