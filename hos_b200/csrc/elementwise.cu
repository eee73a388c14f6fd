// Memory-bound kernels around the matrix products: embedding, RMSNorm and its
// fusions with the residual sum, rotary encoding fused with the cache write,
// the gated activation, row gather.  Statistics, angles and the residual sum are
// 32-bit; only what a matrix product reads next is rounded to the activation type.
#include "common.cuh"
#include "kv_layout.cuh"

namespace hos {

// ---- embedding ---------------------------------------------------------------------
// out[n, :] = table[token[n], :] * scale   (32-bit multiply; a negative token id,
// which marks padding, gives a zero row).
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float scale, float* __restrict__ out, int D) {
    pdl_enter();      // the kernels before this one are complete from here on
    const int n = blockIdx.x;
    const int tok = tokens[n];
    float* o = out + (size_t)n * D;
    if (tok < 0) {
        for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = 0.f;
        return;
    }
    const TW* row = table + (size_t)tok * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = to_float(row[d]) * scale;
}

// ---- RMSNorm -----------------------------------------------------------------------
// y = x * rsqrt(mean(x^2) + eps) * (w + add_one).  One block per row; the row is
// held in shared memory between the two passes.
template <typename TIn, typename TOut>
__global__ void rmsnorm_kernel(const TIn* __restrict__ x, const float* __restrict__ w, float eps,
                               float add_one, TOut* __restrict__ out, int D) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = to_float(x[base + d]);
        row[d] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        out[base + d] = from_float<TOut>(row[d] * r * (w[d] + add_one));
}

// x += RMSNorm(y; w_post);  optionally h = RMSNorm(x; w_next).
// The sandwich arrangement's "post norm, residual sum, next pre norm" in one pass
// over the row: y is read once, x is read and written once, h is written once.
template <typename TY, typename TH>
__global__ void norm_add_norm_kernel(const TY* __restrict__ y, const float* __restrict__ w_post,
                                     float eps_post, float add_one_post, float* __restrict__ x,
                                     const float* __restrict__ w_next, float eps_next,
                                     float add_one_next, TH* __restrict__ h, int D) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = to_float(y[base + d]);
        row[d] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + eps_post);
    float ss2 = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = x[base + d] + row[d] * r * (w_post[d] + add_one_post);
        x[base + d] = v;
        row[d] = v;
        ss2 += v * v;
    }
    if (h == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)D + eps_next);
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        h[base + d] = from_float<TH>(row[d] * r2 * (w_next[d] + add_one_next));
}

// ---- the same two norms with the row in registers ---------------------------------------
// For widths that are a multiple of 4 and fit CH chunks of 4 per thread: every load is issued
// before the first reduction, nothing goes through shared memory but the two block sums.
// `y` may be given as n_parts partial sums of 32-bit floats, [n_parts][rows][D] (what a
// matrix product that split K leaves): they are added here, in a fixed order.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename TIn, typename TOut, int CH>
__global__ void rmsnorm_vec_kernel(const TIn* __restrict__ x, const float* __restrict__ w, float eps,
                                   float add_one, TOut* __restrict__ out, int D) {
    pdl_enter();      // the kernels before this one are complete from here on
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float4 xv[CH], wv[CH];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < D) {
            xv[c] = load4(x + base + i);
            wv[c] = load4(w + i);
            ss += xv[c].x * xv[c].x + xv[c].y * xv[c].y + xv[c].z * xv[c].z + xv[c].w * xv[c].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < D)
            store4(out + base + i, make_float4(xv[c].x * r * (wv[c].x + add_one), xv[c].y * r * (wv[c].y + add_one),
                                               xv[c].z * r * (wv[c].z + add_one), xv[c].w * r * (wv[c].w + add_one)));
    }
}

template <typename TY, typename TH, int CH>
__global__ void norm_add_norm_vec_kernel(const TY* __restrict__ y, int n_parts, size_t part_stride,
                                         const float* __restrict__ w_post, float eps_post, float add_one_post,
                                         float* __restrict__ x, const float* __restrict__ w_next, float eps_next,
                                         float add_one_next, TH* __restrict__ h, int D, int late_flag) {
    // This kernel may be launched ahead of the end of the kernel before it (a few rows: decoding): its CTAs
    // are placed and the norms' weights, which no kernel writes, are fetched meanwhile.  Then (`late_flag`) it lets
    // the kernel after it go only when the kernel before it has ended: a chain of kernels that all wait on the SMs
    // costs more than it hides.
    const bool late_x = late_flag != 0;
    if (!late_x) pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * D;
    float4 yv[CH], xv[CH], wp[CH], wn[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < D) {
            wp[c] = load4(w_post + i);
            if (h != nullptr) wn[c] = load4(w_next + i);
        }
    }
    pdl_wait();       // the kernels before this one are complete from here on
    if (late_x) pdl_launch_dependents();
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < D) {
            yv[c] = load4(y + base + i);
            for (int p = 1; p < n_parts; ++p) {
                const float4 t = load4(y + p * part_stride + base + i);
                yv[c].x += t.x; yv[c].y += t.y; yv[c].z += t.z; yv[c].w += t.w;
            }
            xv[c] = load4(x + base + i);
            ss += yv[c].x * yv[c].x + yv[c].y * yv[c].y + yv[c].z * yv[c].z + yv[c].w * yv[c].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)D + eps_post);
    float ss2 = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < D) {
            xv[c].x += yv[c].x * r * (wp[c].x + add_one_post);
            xv[c].y += yv[c].y * r * (wp[c].y + add_one_post);
            xv[c].z += yv[c].z * r * (wp[c].z + add_one_post);
            xv[c].w += yv[c].w * r * (wp[c].w + add_one_post);
            store4(x + base + i, xv[c]);
            ss2 += xv[c].x * xv[c].x + xv[c].y * xv[c].y + xv[c].z * xv[c].z + xv[c].w * xv[c].w;
        }
    }
    if (h == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.0f / sqrtf(ss2 / (float)D + eps_next);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < D)
            store4(h + base + i, make_float4(xv[c].x * r2 * (wn[c].x + add_one_next), xv[c].y * r2 * (wn[c].y + add_one_next),
                                             xv[c].z * r2 * (wn[c].z + add_one_next), xv[c].w * r2 * (wn[c].w + add_one_next)));
    }
}

// ---- the same for many rows (a prompt) -----------------------------------------------------
// A CTA of D/8 threads walks over rows (row = blockIdx.x, += gridDim.x); a thread owns 8 columns,
// keeps the two norms' weights for them in registers for all its rows, and issues the loads of its
// next row before it reduces the current one, so that the two block sums of a row do not leave
// the memory pipe empty.  bfloat16 branch output and next-norm output, 32-bit residual stream.
constexpr int kRowsKernelMinRows = 256;
struct Row8 { float v[8]; };
__device__ __forceinline__ Row8 load8(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    return Row8{{a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w}};
}
__device__ __forceinline__ Row8 load8(const bf16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
    Row8 r;
#pragma unroll
    for (int i = 0; i < 4; ++i) { r.v[2 * i] = __low2float(h2[i]); r.v[2 * i + 1] = __high2float(h2[i]); }
    return r;
}
__device__ __forceinline__ void store8(float* p, const Row8& r) {
    *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(r.v[4], r.v[5], r.v[6], r.v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const Row8& r) {
    uint4 u;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(r.v[2 * i], r.v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}

template <typename TY, typename TH>
__global__ void norm_add_norm_rows_kernel(const TY* __restrict__ y, int n_parts, size_t part_stride,
                                          const float* __restrict__ w_post, float eps_post, float add_one_post,
                                          float* __restrict__ x, const float* __restrict__ w_next, float eps_next,
                                          float add_one_next, TH* __restrict__ h, int D, int N) {
    // launched ahead of the end of the kernel before it: the CTAs are placed and the norms' weights, which no
    // kernel writes, are fetched meanwhile
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const int c0 = threadIdx.x * 8;
    const bool live = c0 < D;                       // the block is rounded up to whole warps
    Row8 wp, wn;
#pragma unroll
    for (int i = 0; i < 8; ++i) wp.v[i] = wn.v[i] = 0.f;
    if (live) {
        wp = load8(w_post + c0);
        if (h != nullptr) wn = load8(w_next + c0);
    }
    pdl_wait();       // the kernels before this one are complete from here on
    auto fetch_y = [&](int row) {
        Row8 r = load8(y + (size_t)row * D + c0);
        for (int p = 1; p < n_parts; ++p) {
            const Row8 t = load8(y + p * part_stride + (size_t)row * D + c0);
#pragma unroll
            for (int i = 0; i < 8; ++i) r.v[i] += t.v[i];
        }
        return r;
    };
    int row = blockIdx.x;
    Row8 yv, xv;
#pragma unroll
    for (int i = 0; i < 8; ++i) yv.v[i] = xv.v[i] = 0.f;
    if (row < N && live) { yv = fetch_y(row); xv = load8(x + (size_t)row * D + c0); }
    while (row < N) {
        const int next = row + gridDim.x;
        Row8 yn = yv, xn = xv;
        if (next < N && live) { yn = fetch_y(next); xn = load8(x + (size_t)next * D + c0); }   // in flight during the sums
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += yv.v[i] * yv.v[i];
        ss = block_sum(ss, scratch);
        const float r = 1.0f / sqrtf(ss / (float)D + eps_post);
        float ss2 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            xv.v[i] += yv.v[i] * r * (wp.v[i] + add_one_post);
            ss2 += xv.v[i] * xv.v[i];
        }
        if (live) store8(x + (size_t)row * D + c0, xv);
        if (h != nullptr) {
            ss2 = block_sum(ss2, scratch);
            const float r2 = 1.0f / sqrtf(ss2 / (float)D + eps_next);
            Row8 o;
#pragma unroll
            for (int i = 0; i < 8; ++i) o.v[i] = xv.v[i] * r2 * (wn.v[i] + add_one_next);
            if (live) store8(h + (size_t)row * D + c0, o);
        }
        yv = yn; xv = xn; row = next;
    }
}

// Threads per row and chunks per thread for the register-resident kernels; chunks 0: use the others.
static void vec_shape(int D, int* threads, int* chunks) {
    *chunks = 0;
    if (D % 4 != 0) return;
    const int quads = D / 4;
    for (int ch = 1; ch <= 4; ch *= 2) {
        if (quads <= 1024 * ch) {
            *chunks = ch;
            *threads = (((quads + ch - 1) / ch) + 31) / 32 * 32;
            return;
        }
    }
}

// x += y (plain residual sum in 32-bit, for arrangements without a post norm).
template <typename TY>
__global__ void residual_add_kernel(const TY* __restrict__ y, float* __restrict__ x, size_t n) {
    pdl_enter();      // the kernels before this one are complete from here on
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_float(y[i]);
}

// ---- the angles of a step, once for all layers -------------------------------------------------
// out[n][i] = (cos, sin) of position[n] * inv_freq[i], in 32-bit: what the q/k/v projection of many tokens
// reads in its epilogue instead of taking a sine and a cosine per head.
__global__ void rope_table_kernel(const int* __restrict__ token_pos, const float* __restrict__ inv_freq,
                                  float2* __restrict__ out, int N, int half) {
    pdl_enter();      // the kernels before this one are complete from here on
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)N * half) return;
    const int n = (int)(idx / half), i = (int)(idx % half);
    float sn, cs;
    sincosf((float)token_pos[n] * inv_freq[i], &sn, &cs);
    out[idx] = make_float2(cs, sn);
}

// ---- rotary encoding + cache write --------------------------------------------------
// One block per token.  The q and k heads of the fused projection row are rotated
// (angle = position * inv_freq[i], sincosf in 32-bit, once per pair and token), the row is
// left in `qkv` as the activation type, and the rotated key and the value go to the token's
// place in the paged cache.  The source is `qkv` itself (rotation in place) or n_parts
// partial sums of 32-bit floats [n_parts][rows][row_stride] from a matrix product that split
// K, added here in a fixed order.  A token whose place in a ring is overwritten by a later
// token of the same step is not stored.
// style 0: pairs (i, i + rot/2) ("rotate half"); style 1: pairs (2i, 2i+1).
template <typename TSrc, typename T>
__global__ void rope_kv_write_kernel(const TSrc* __restrict__ src, int n_parts, size_t part_stride,
                                     T* __restrict__ qkv, int row_stride, int n_heads,
                                     const int* __restrict__ token_pos,
                                     const int* __restrict__ token_seq,
                                     const int* __restrict__ seq_slot,
                                     const int* __restrict__ seq_len_after,
                                     const float* __restrict__ inv_freq, int rotary_dim, int style,
                                     PagedKV cache, int write_cache) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ float2 sincos_tab[];          // [rotary_dim / 2]
    const int n = blockIdx.x;
    const int seq = token_seq[n];
    if (seq < 0) return;
    const int pos = token_pos[n];
    const int hd = cache.head_dim, nkv = cache.n_kv_heads;
    const int half = rotary_dim >> 1;
    // where the token's key and value go: looked up now, so that these dependent loads overlap the rotation
    int page = -1;
    if (write_cache && !(cache.ring_pages > 0 && pos + cache.ring_pages * kPageTokens < seq_len_after[seq]))
        page = cache.page_table[(size_t)seq_slot[seq] * cache.table_stride + kv_table_entry(cache, pos / kPageTokens)];
    const bool in_place = (const void*)src == (const void*)qkv;
    const TSrc* srow = src + (size_t)n * row_stride;
    T* row = qkv + (size_t)n * row_stride;
    auto value = [&](int e) {
        float v = to_float(srow[e]);
        for (int p = 1; p < n_parts; ++p) v += to_float(srow[p * part_stride + e]);
        return v;
    };
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sincos_tab[i] = make_float2(s, c);
    }
    __syncthreads();
    // heads [0, n_heads) are q, [n_heads, n_heads + nkv) are k, then nkv heads of v
    const int n_rot_heads = n_heads + nkv;
    for (int idx = threadIdx.x; idx < n_rot_heads * half; idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        const int a = style == 0 ? i : 2 * i;
        const int b = style == 0 ? i + half : 2 * i + 1;
        const float2 sc = sincos_tab[i];
        const float x0 = value(head * hd + a), x1 = value(head * hd + b);
        row[head * hd + a] = from_float<T>(x0 * sc.y - x1 * sc.x);
        row[head * hd + b] = from_float<T>(x0 * sc.x + x1 * sc.y);
    }
    if (!in_place) {      // what is not rotated still has to reach the activation row
        const int pass = hd - rotary_dim;
        for (int idx = threadIdx.x; idx < n_rot_heads * pass; idx += blockDim.x) {
            const int head = idx / pass, d = rotary_dim + idx % pass;
            row[head * hd + d] = from_float<T>(value(head * hd + d));
        }
        for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
            const int e = (n_heads + nkv) * hd + idx;
            row[e] = from_float<T>(value(e));
        }
    }
    if (page < 0) return;          // nothing to store (no cache, or a ring position that this step overwrites)
    __syncthreads();
    const int r = pos % kPageTokens;
    const T* ksrc = row + (size_t)n_heads * hd;
    const T* vsrc = ksrc + (size_t)nkv * hd;
    T* kp = (T*)cache.k_pages;
    T* vp = (T*)cache.v_pages;
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int kvh = idx / hd, d = idx - kvh * hd;
        const size_t off = kv_tile_offset(cache, page, kvh) + kv_elem_offset(r, d, hd);
        kp[off] = ksrc[idx];
        vp[off] = vsrc[idx];
    }
}

// The same for bfloat16 rows rotated in place, 16 bytes at a time: a thread takes a chunk of 8
// elements of a head (and, for the rotate-half pairing, its partner chunk half a rotation
// away), rotates it, writes it back and, if it belongs to a key, also to the cache; value
// chunks and unrotated key chunks are copied to the cache.  One pass, one barrier (for the
// table of sines and cosines); the look-ups that lead to the token's page run beside it.
// Needs head_dim % 8 == 0 and rotary_dim % 16 == 0 (rotate-half) or % 8 == 0 (interleaved).
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(p[i]); f[2 * i + 1] = __high2float(p[i]); }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

// PARTS: the rows come as n_parts partial sums of 32-bit floats (what a matrix product that split K
// leaves) and are formed here; everything, rotated or not, is then written to the bfloat16 row.
// Otherwise the bfloat16 rows are rotated in place.  gridDim.y CTAs share a token's chunks.
template <bool PARTS>
__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(const float* __restrict__ parts, int n_parts, size_t part_stride,
                         bf16* __restrict__ qkv, int row_stride, int n_heads,
                         const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_len_after,
                         const float* __restrict__ inv_freq, int rotary_dim, int style,
                         PagedKV cache, int write_cache) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ float2 sincos_tab[];          // [rotary_dim / 2]
    const int n = blockIdx.x;
    const int seq = token_seq[n];
    if (seq < 0) return;
    const int pos = token_pos[n];
    const int hd = cache.head_dim, nkv = cache.n_kv_heads;
    const int half = rotary_dim >> 1;
    int page = -1;
    if (write_cache && !(cache.ring_pages > 0 && pos + cache.ring_pages * kPageTokens < seq_len_after[seq]))
        page = cache.page_table[(size_t)seq_slot[seq] * cache.table_stride + kv_table_entry(cache, pos / kPageTokens)];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sincos_tab[i] = make_float2(s, c);
    }
    __syncthreads();
    bf16* row = qkv + (size_t)n * row_stride;
    const float* prow = PARTS ? parts + (size_t)n * row_stride : nullptr;
    // 8 elements of the row from element e on, as floats
    auto fetch = [&](int e, float (&f)[8]) {
        if (PARTS) {
            const float4 a = *reinterpret_cast<const float4*>(prow + e), b2 = *reinterpret_cast<const float4*>(prow + e + 4);
            f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b2.x; f[5] = b2.y; f[6] = b2.z; f[7] = b2.w;
            for (int p = 1; p < n_parts; ++p) {
                const float4 c = *reinterpret_cast<const float4*>(prow + p * part_stride + e);
                const float4 d = *reinterpret_cast<const float4*>(prow + p * part_stride + e + 4);
                f[0] += c.x; f[1] += c.y; f[2] += c.z; f[3] += c.w; f[4] += d.x; f[5] += d.y; f[6] += d.z; f[7] += d.w;
            }
        } else {
            unpack8(*reinterpret_cast<const uint4*>(row + e), f);
        }
    };
    bf16* kp = (bf16*)cache.k_pages;
    bf16* vp = (bf16*)cache.v_pages;
    const int r = pos % kPageTokens;
    const int chunks = hd / 8;                                  // 16-byte chunks per head
    const int rot_chunks = rotary_dim / 8;
    const int rot_items = style == 0 ? rot_chunks / 2 : rot_chunks;   // rotate-half: a chunk and its partner
    const int tail_chunks = chunks - rot_chunks;
    const int per_qk_head = rot_items + tail_chunks;
    const int n_qk = n_heads + nkv;
    const int total = n_qk * per_qk_head + nkv * chunks;
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < total; item += gridDim.y * blockDim.x) {
        if (item < n_qk * per_qk_head) {
            const int head = item / per_qk_head, j = item % per_qk_head;
            const int h0 = head * hd;
            const bool is_k = head >= n_heads;
            const size_t tile = is_k && page >= 0 ? kv_tile_offset(cache, page, head - n_heads) : 0;
            float fa[8], fb[8];
            if (j >= rot_items) {                                // beyond the rotated dimensions: as they are
                const int d0 = rotary_dim + (j - rot_items) * 8;
                if (!PARTS && !(is_k && page >= 0)) continue;
                fetch(h0 + d0, fa);
                const uint4 oa = pack8(fa);
                if (PARTS) *reinterpret_cast<uint4*>(row + h0 + d0) = oa;
                if (is_k && page >= 0) *reinterpret_cast<uint4*>(kp + tile + kv_elem_offset(r, d0, hd)) = oa;
                continue;
            }
            if (style == 0) {
                const int da = j * 8, db = half + j * 8;
                fetch(h0 + da, fa); fetch(h0 + db, fb);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float2 sc = sincos_tab[j * 8 + e];
                    const float x0 = fa[e], x1 = fb[e];
                    fa[e] = x0 * sc.y - x1 * sc.x;
                    fb[e] = x0 * sc.x + x1 * sc.y;
                }
                const uint4 oa = pack8(fa), ob = pack8(fb);
                *reinterpret_cast<uint4*>(row + h0 + da) = oa;
                *reinterpret_cast<uint4*>(row + h0 + db) = ob;
                if (is_k && page >= 0) {
                    *reinterpret_cast<uint4*>(kp + tile + kv_elem_offset(r, da, hd)) = oa;
                    *reinterpret_cast<uint4*>(kp + tile + kv_elem_offset(r, db, hd)) = ob;
                }
            } else {
                const int d0 = j * 8;
                fetch(h0 + d0, fa);
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float2 sc = sincos_tab[(d0 + e) >> 1];
                    const float x0 = fa[e], x1 = fa[e + 1];
                    fa[e] = x0 * sc.y - x1 * sc.x;
                    fa[e + 1] = x0 * sc.x + x1 * sc.y;
                }
                const uint4 oa = pack8(fa);
                *reinterpret_cast<uint4*>(row + h0 + d0) = oa;
                if (is_k && page >= 0) *reinterpret_cast<uint4*>(kp + tile + kv_elem_offset(r, d0, hd)) = oa;
            }
        } else if (PARTS || page >= 0) {
            const int v = item - n_qk * per_qk_head;
            const int kvh = v / chunks, d0 = (v % chunks) * 8;
            const int e0 = (n_heads + nkv + kvh) * hd + d0;
            float fv[8];
            fetch(e0, fv);
            const uint4 ov = pack8(fv);
            if (PARTS) *reinterpret_cast<uint4*>(row + e0) = ov;
            if (page >= 0) *reinterpret_cast<uint4*>(vp + kv_tile_offset(cache, page, kvh) + kv_elem_offset(r, d0, hd)) = ov;
        }
    }
}

// ---- gated activation ---------------------------------------------------------------
// out[n, f] = act(gu[n, f]) * gu[n, F + f]; act 0 = tanh-form GELU, 1 = SiLU.
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, int act) {
    pdl_enter();      // the kernels before this one are complete from here on
    const size_t n = blockIdx.x;
    const int f = blockIdx.y * blockDim.x + threadIdx.x;
    if (f >= F) return;
    const float g = to_float(gu[n * 2 * F + f]);
    const float u = to_float(gu[n * 2 * F + F + f]);
    const float a = act == 0 ? gelu_tanh(g) : g / (1.f + expf(-g));
    out[n * F + f] = from_float<T>(a * u);
}

// ---- row gather ----------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ idx,
                                   float* __restrict__ out, int D) {
    pdl_enter();      // the kernels before this one are complete from here on
    const int i = blockIdx.x;
    const float* src = x + (size_t)idx[i] * D;
    float* dst = out + (size_t)i * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
}

// After a decode step whose tokens were chosen on the device: the chosen token becomes
// the next step's input, positions and lengths move on by one (padding rows stay as they are).
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ token_pos,
                                      int* __restrict__ seq_len_after, const int* __restrict__ token_seq,
                                      const int* __restrict__ sampled, int B) {
    pdl_enter();      // the kernels before this one are complete from here on
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B || token_seq[i] < 0) return;
    tokens[i] = sampled[i];
    token_pos[i] += 1;
    seq_len_after[i] += 1;
}

static int row_smem_ok(const void* kernel, int D) {
    size_t bytes = (size_t)D * sizeof(float);
    if (bytes > 200 * 1024) return -1;
    if (bytes > 48 * 1024)
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return 0;
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

extern "C" int hos_embed(const int* tokens, const void* table, int table_dtype, float scale,
                         float* out, int N, int D, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (table_dtype == kBF16)
        launch_pdl(embed_kernel<bf16>, dim3(N), dim3(256), 0, stream, tokens, (const bf16*)table, scale, out, D);
    else if (table_dtype == kF32)
        launch_pdl(embed_kernel<float>, dim3(N), dim3(256), 0, stream, tokens, (const float*)table, scale, out, D);
    else
        HOS_REFUSE("embed: unknown table dtype %d", table_dtype);
    return check_launch("embed");
}

extern "C" int hos_rmsnorm(const void* x, int x_dtype, const float* w, float eps, int add_one,
                           void* out, int out_dtype, int N, int D, cudaStream_t stream) {
    if (N <= 0) return 0;
    const size_t smem = (size_t)D * sizeof(float);
    const float a1 = add_one ? 1.f : 0.f;
    int threads = 0, chunks = 0;
    vec_shape(D, &threads, &chunks);
    if (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w) % 16) chunks = 0;
#define HOS_VEC(TI, TO, CH) launch_pdl(rmsnorm_vec_kernel<TI, TO, CH>, dim3(N), dim3(threads), 0, stream, (const TI*)x, w, eps, a1, (TO*)out, D)
#define HOS_LAUNCH_NORM(TI, TO)                                                              \
    do {                                                                                     \
        if (chunks == 1) HOS_VEC(TI, TO, 1);                                                 \
        else if (chunks == 2) HOS_VEC(TI, TO, 2);                                            \
        else if (chunks == 4) HOS_VEC(TI, TO, 4);                                            \
        else {                                                                               \
            if (row_smem_ok((const void*)rmsnorm_kernel<TI, TO>, D))                         \
                HOS_REFUSE("rmsnorm: width %d does not fit a block's shared memory", D);     \
            launch_pdl(rmsnorm_kernel<TI, TO>, dim3(N), dim3(256), smem, stream, (const TI*)x, w, eps, a1, (TO*)out, D); \
        }                                                                                    \
    } while (0)
    if (x_dtype == kF32 && out_dtype == kF32) HOS_LAUNCH_NORM(float, float);
    else if (x_dtype == kF32 && out_dtype == kBF16) HOS_LAUNCH_NORM(float, bf16);
    else if (x_dtype == kBF16 && out_dtype == kBF16) HOS_LAUNCH_NORM(bf16, bf16);
    else if (x_dtype == kBF16 && out_dtype == kF32) HOS_LAUNCH_NORM(bf16, float);
    else HOS_REFUSE("rmsnorm: unknown dtypes %d -> %d", x_dtype, out_dtype);
#undef HOS_LAUNCH_NORM
#undef HOS_VEC
    return check_launch("rmsnorm");
}

// x += RMSNorm(y; w_post); if h != NULL also h = RMSNorm(x; w_next), written as h_dtype.
// n_parts > 1: y is n_parts partial sums of 32-bit floats, [n_parts][N][D], added here.
extern "C" int hos_norm_add_norm(const void* y, int y_dtype, int n_parts, const float* w_post, float eps_post,
                                 int add_one_post, float* x, const float* w_next, float eps_next,
                                 int add_one_next, void* h, int h_dtype, int N, int D, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_parts < 1 || (n_parts > 1 && y_dtype != kF32))
        HOS_REFUSE("norm_add_norm: partial sums are 32-bit floats (n_parts %d, dtype %d)", n_parts, y_dtype);
    const size_t smem = (size_t)D * sizeof(float);
    const float a1 = add_one_post ? 1.f : 0.f, a2 = add_one_next ? 1.f : 0.f;
    const size_t ps = (size_t)N * D;
    int threads = 0, chunks = 0;
    vec_shape(D, &threads, &chunks);
    if (((uintptr_t)y | (uintptr_t)x | (uintptr_t)h | (uintptr_t)w_post | (uintptr_t)w_next) % 16) chunks = 0;
    if (chunks == 0 && n_parts > 1) HOS_REFUSE("norm_add_norm: partial sums need a width that is a multiple of 4 (%d)", D);
    // A few rows (decoding): the kernel is launched ahead of the end of the product before it, so that its CTAs are
    // placed and the norms' weights fetched while that one finishes (a batch-8 step 2.154 -> 2.129 ms, one sequence
    // 1.533 -> 1.503 ms, 64 sequences 8.098 -> 8.090 ms); HOS_NORM_AHEAD=0 switches it off.
    static const bool few_rows_ahead = !(getenv("HOS_NORM_AHEAD") && getenv("HOS_NORM_AHEAD")[0] == '0');
    const bool ahead = pdl_enabled() || (few_rows_ahead && N < kRowsKernelMinRows);
    const int norm_late = ahead ? 1 : 0;
#define HOS_VEC(TY, TH, CH) launch_ahead(ahead, norm_add_norm_vec_kernel<TY, TH, CH>, dim3(N), dim3(threads), 0, stream,         \
        (const TY*)y, n_parts, ps, w_post, eps_post, a1, x, w_next, eps_next, a2, (TH*)h, D, norm_late)
#define HOS_LAUNCH(TY, TH)                                                                                  \
    do {                                                                                                    \
        if (chunks == 1) HOS_VEC(TY, TH, 1);                                                                \
        else if (chunks == 2) HOS_VEC(TY, TH, 2);                                                           \
        else if (chunks == 4) HOS_VEC(TY, TH, 4);                                                           \
        else {                                                                                              \
            if (row_smem_ok((const void*)norm_add_norm_kernel<TY, TH>, D))                                  \
                HOS_REFUSE("norm_add_norm: width %d does not fit a block's shared memory", D);              \
            launch_pdl(norm_add_norm_kernel<TY, TH>, dim3(N), dim3(256), smem, stream,                                          \
                (const TY*)y, w_post, eps_post, a1, x, w_next, eps_next, a2, (TH*)h, D);                    \
        }                                                                                                   \
    } while (0)
    if (h == nullptr) h_dtype = y_dtype == kF32 ? kF32 : kBF16;
    // many rows of a width in steps of 8: CTAs that walk over rows with the next row's loads in flight
    if (N >= kRowsKernelMinRows && chunks != 0 && D % 8 == 0 && D / 8 <= 1024) {
        const int threads_r = (D / 8 + 31) / 32 * 32;
        // about 1024 threads per SM: measured best (3 CTAs of 288 threads at width 2304; more CTAs with fewer rows each
        // lose what the loads in flight across the sums gain)
        const int per_sm = 1024 / threads_r < 1 ? 1 : 1024 / threads_r;
        const int grid_r = N < sm_count_cached() * per_sm ? N : sm_count_cached() * per_sm;
#define HOS_ROWS(TY, TH) launch_pdl(norm_add_norm_rows_kernel<TY, TH>, dim3(grid_r), dim3(threads_r), 0, stream,            \
        (const TY*)y, n_parts, ps, w_post, eps_post, a1, x, w_next, eps_next, a2, (TH*)h, D, N)
        if (y_dtype == kF32 && h_dtype == kF32) HOS_ROWS(float, float);
        else if (y_dtype == kF32 && h_dtype == kBF16) HOS_ROWS(float, bf16);
        else if (y_dtype == kBF16 && h_dtype == kBF16) HOS_ROWS(bf16, bf16);
        else HOS_REFUSE("norm_add_norm: no kernel for dtypes %d -> %d", y_dtype, h_dtype);
#undef HOS_ROWS
        return check_launch("norm_add_norm");
    }
    if (y_dtype == kF32 && h_dtype == kF32) HOS_LAUNCH(float, float);
    else if (y_dtype == kF32 && h_dtype == kBF16) HOS_LAUNCH(float, bf16);
    else if (y_dtype == kBF16 && h_dtype == kBF16) HOS_LAUNCH(bf16, bf16);
    else HOS_REFUSE("norm_add_norm: no kernel for dtypes %d -> %d", y_dtype, h_dtype);
#undef HOS_LAUNCH
#undef HOS_VEC
    return check_launch("norm_add_norm");
}

extern "C" int hos_residual_add(const void* y, int y_dtype, float* x, long long n,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (y_dtype == kF32) launch_pdl(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)y, x, (size_t)n);
    else if (y_dtype == kBF16) launch_pdl(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)y, x, (size_t)n);
    else HOS_REFUSE("residual_add: unknown dtype %d", y_dtype);
    return check_launch("residual_add");
}

// src_dtype/n_parts: the source of the rows; src == qkv (same dtype, n_parts 1) rotates in place,
// a 32-bit source with n_parts >= 1 is summed over its parts and written to qkv.
extern "C" int hos_rope_kv_write(const void* src, int src_dtype, int n_parts, void* qkv, int dtype,
                                 int row_stride, int n_heads,
                                 const int* token_pos, const int* token_seq, const int* seq_slot,
                                 const int* seq_len_after, const float* inv_freq, int rotary_dim,
                                 int style, void* k_pages, void* v_pages, const int* page_table,
                                 int table_stride, int ring_pages, int n_kv_heads, int head_dim,
                                 int write_cache, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        HOS_REFUSE("rope: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    if (style != 0 && style != 1) HOS_REFUSE("rope: unknown pairing style %d", style);
    if (n_parts < 1 || (src != qkv && src_dtype != kF32) || (src == qkv && (n_parts != 1 || src_dtype != dtype)))
        HOS_REFUSE("rope: the source is the rows themselves or 32-bit partial sums");
    PagedKV c{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim};
    const size_t smem = (size_t)(rotary_dim / 2) * sizeof(float2);
    const size_t ps = (size_t)N * row_stride;
#define HOS_ROPE(TS, T)                                                                              \
    launch_pdl(rope_kv_write_kernel<TS, T>, dim3(N), dim3(256), smem, stream, (const TS*)src, n_parts, ps, (T*)qkv, row_stride, \
        n_heads, token_pos, token_seq, seq_slot, seq_len_after, inv_freq, rotary_dim, style, c, write_cache)
    const bool from_parts = src != qkv;             // then src_dtype is kF32 (checked above)
    const bool vec_ok = dtype == kBF16 && (head_dim % 8) == 0 && (row_stride % 8) == 0 &&
                        ((uintptr_t)qkv % 16) == 0 && (rotary_dim % (style == 0 ? 16 : 8)) == 0 &&
                        (!from_parts || (((uintptr_t)src % 16) == 0 && (ps % 4) == 0)) &&
                        (!write_cache || (((uintptr_t)k_pages | (uintptr_t)v_pages) % 16) == 0);
    if (vec_ok) {
        // few tokens: several CTAs share a token's chunks, so that the launch fills more of the GPU
        const int chunks_per_token = (n_heads + 2 * n_kv_heads) * (head_dim / 8);
        int share = 1;
        while (share < 8 && N * share < 2 * sm_count_cached() && chunks_per_token / (share * 2) >= 128) share *= 2;
        if (from_parts)
            launch_pdl(rope_kv_write_vec_kernel<true>, dim3(N, share), dim3(256), smem, stream, (const float*)src, n_parts, ps,
                (bf16*)qkv, row_stride, n_heads, token_pos, token_seq, seq_slot, seq_len_after, inv_freq, rotary_dim, style, c,
                write_cache);
        else
            launch_pdl(rope_kv_write_vec_kernel<false>, dim3(N, share), dim3(256), smem, stream, (const float*)nullptr, 1, ps,
                (bf16*)qkv, row_stride, n_heads, token_pos, token_seq, seq_slot, seq_len_after, inv_freq, rotary_dim, style, c,
                write_cache);
        return check_launch("rope_kv_write");
    }
    if (dtype == kF32) HOS_ROPE(float, float);
    else if (dtype == kBF16 && src_dtype == kBF16) HOS_ROPE(bf16, bf16);
    else if (dtype == kBF16 && src_dtype == kF32) HOS_ROPE(float, bf16);
    else HOS_REFUSE("rope: unknown dtype %d", dtype);
#undef HOS_ROPE
    return check_launch("rope_kv_write");
}

extern "C" int hos_rope_table(const int* token_pos, const float* inv_freq, float* out, int N, int half,
                              cudaStream_t stream) {
    if (N <= 0 || half <= 0) return 0;
    const size_t n = (size_t)N * half;
    launch_pdl(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, token_pos, inv_freq,
               reinterpret_cast<float2*>(out), N, half);
    return check_launch("rope_table");
}

extern "C" int hos_gated_act(const void* gu, void* out, int dtype, int N, int F, int act,
                             cudaStream_t stream) {
    if (N <= 0) return 0;
    if (act != 0 && act != 1) HOS_REFUSE("gated_act: unknown activation %d", act);
    dim3 grid(N, (F + 255) / 256);
    if (dtype == kF32) launch_pdl(gated_act_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)gu, (float*)out, F, act);
    else if (dtype == kBF16) launch_pdl(gated_act_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, F, act);
    else HOS_REFUSE("gated_act: unknown dtype %d", dtype);
    return check_launch("gated_act");
}

extern "C" int hos_gather_rows(const float* x, const int* idx, float* out, int n, int D,
                               cudaStream_t stream) {
    if (n <= 0) return 0;
    launch_pdl(gather_rows_kernel, dim3(n), dim3(256), 0, stream, x, idx, out, D);
    return check_launch("gather_rows");
}

extern "C" int hos_decode_advance(int* tokens, int* token_pos, int* seq_len_after, const int* token_seq,
                                  const int* sampled, int B, cudaStream_t stream) {
    if (B <= 0) return 0;
    launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, token_pos, seq_len_after,
                                                               token_seq, sampled, B);
    return check_launch("decode_advance");
}
