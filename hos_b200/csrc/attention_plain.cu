// Plain attention: one warp per (token, query head), keys visited one by one with a
// running maximum and sum, everything in 32-bit with precise tanhf and expf.  Any
// head size up to 1024, any number of heads and groups.  It is the 32-bit path's
// attention, the reference of the tensor-core attention kernels, and the kernel for
// cases those refuse (a layer that reads another call's cache during a prompt).
//
// Two sources of keys: the rows of this step's own packed projection output (a
// prompt from position 0: nothing is read from the cache), or the paged cache.
// Scores: (q.k) * scale, soft-capped, keys t in [max(0, pos + 1 - window), pos]
// (window <= 0: all keys up to pos), softmax, weighted sum of values.
#include "common.cuh"
#include "kv_layout.cuh"

namespace hos {

constexpr int kMaxPerLane = 32;   // head_dim <= 32 * kMaxPerLane

template <typename T, bool PAGED, int PL>
__global__ void __launch_bounds__(128)
attn_plain_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_rows,
                  const T* __restrict__ v_rows, int kv_stride, T* __restrict__ out, int out_stride,
                  const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                  PagedKV cache, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                  float scale, float cap, int window) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int n = (int)(item / n_heads), h = (int)(item % n_heads);
    constexpr int per_lane = PL;   // head_dim <= 32 * PL
    T* o = out + (size_t)n * out_stride + (size_t)h * head_dim;
    const int seq = token_seq[n];
    if (seq < 0) {   // padding: defined output, no reads
        for (int i = 0; i < per_lane; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) o[d] = from_float<T>(0.f);
        }
        return;
    }
    const int pos = token_pos[n];
    const int kvh = h / (n_heads / n_kv_heads);
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;

    float qreg[PL], acc[PL];
    const T* qp = q + (size_t)n * q_stride + (size_t)h * head_dim;
#pragma unroll
    for (int i = 0; i < per_lane; ++i) {
        const int d = lane + 32 * i;
        qreg[i] = d < head_dim ? to_float(qp[d]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int slot = PAGED ? seq_slot[seq] : 0;
    const size_t row0 = PAGED ? 0 : (size_t)cu_seqlens[seq];

    for (int t = lo; t <= pos; ++t) {
        const T* kp;
        const T* vp;
        int r = 0;
        if (PAGED) {
            const int lp = t / kPageTokens;
            r = t % kPageTokens;
            const int page = cache.page_table[(size_t)slot * cache.table_stride + kv_table_entry(cache, lp)];
            const size_t tile = kv_tile_offset(cache, page, kvh);
            kp = (const T*)cache.k_pages + tile;
            vp = (const T*)cache.v_pages + tile;
        } else {
            kp = k_rows + (row0 + t) * kv_stride + (size_t)kvh * head_dim;
            vp = v_rows + (row0 + t) * kv_stride + (size_t)kvh * head_dim;
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < per_lane; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) {
                const int off = PAGED ? kv_elem_offset(r, d, head_dim) : d;
                dot = fmaf(qreg[i], to_float(kp[off]), dot);
            }
        }
        dot = warp_sum(dot);
        const float s = softcap_precise(dot * scale, cap);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);      // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < per_lane; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) {
                const int off = PAGED ? kv_elem_offset(r, d, head_dim) : d;
                acc[i] = acc[i] * corr + p * to_float(vp[off]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < per_lane; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) o[d] = from_float<T>(acc[i] * inv);
    }
}

}  // namespace hos

using namespace hos;

// paged = 0: keys and values are rows of this step (k_rows, v_rows with kv_stride
// elements between tokens, sequence s occupying rows cu_seqlens[s]...), every
// sequence starting at position 0.  paged = 1: keys and values come from the cache.
extern "C" int hos_attn_plain(int dtype, int paged, const void* q, int q_stride, const void* k_rows,
                              const void* v_rows, int kv_stride, void* out, int out_stride,
                              const int* token_pos, const int* token_seq, const int* cu_seqlens,
                              const int* seq_slot, void* k_pages, void* v_pages,
                              const int* page_table, int table_stride, int ring_pages,
                              int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale,
                              float cap, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > 32 * kMaxPerLane)
        HOS_REFUSE("attn_plain: head_dim %d is outside 1..%d", head_dim, 32 * kMaxPerLane);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_plain: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    PagedKV c{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim};
    const long long items = (long long)n_tokens * n_heads;
    const unsigned blocks = (unsigned)((items + 3) / 4);
#define HOS_LAUNCH_PL(T, P, PL)                                                                 \
    attn_plain_kernel<T, P, PL><<<blocks, 128, 0, stream>>>(                                    \
        (const T*)q, q_stride, (const T*)k_rows, (const T*)v_rows, kv_stride, (T*)out,          \
        out_stride, token_pos, token_seq, cu_seqlens, seq_slot, c, n_tokens, n_heads,           \
        n_kv_heads, head_dim, scale, cap, window)
#define HOS_LAUNCH(T, P)                                                                        \
    do {                                                                                        \
        if (head_dim <= 32) HOS_LAUNCH_PL(T, P, 1);                                             \
        else if (head_dim <= 64) HOS_LAUNCH_PL(T, P, 2);                                        \
        else if (head_dim <= 128) HOS_LAUNCH_PL(T, P, 4);                                       \
        else if (head_dim <= 256) HOS_LAUNCH_PL(T, P, 8);                                       \
        else if (head_dim <= 512) HOS_LAUNCH_PL(T, P, 16);                                      \
        else HOS_LAUNCH_PL(T, P, 32);                                                           \
    } while (0)
    if (dtype == kF32 && paged) HOS_LAUNCH(float, true);
    else if (dtype == kF32) HOS_LAUNCH(float, false);
    else if (dtype == kBF16 && paged) HOS_LAUNCH(bf16, true);
    else if (dtype == kBF16) HOS_LAUNCH(bf16, false);
    else HOS_REFUSE("attn_plain: unknown dtype %d", dtype);
#undef HOS_LAUNCH
#undef HOS_LAUNCH_PL
    return check_launch("attn_plain");
}
