// Attention of single tokens over the paged cache (decoding), bfloat16, split over the keys.
//
// One CTA (4 warps) takes one token, one kv head (with the up to 16 query heads that share
// it, stacked as the rows of one MMA tile) and one contiguous share of the sequence's pages.
// A page's [64][HD] key tile and value tile are contiguous in the cache, so one thread brings
// each on chip with a single bulk copy (TMA) counted on an mbarrier, several pages ahead of
// the math.  Per tile each warp takes 16 keys: S = Q K^T (m16n8k16, bf16, 32-bit
// accumulators), scale, soft-cap, mask, running max/sum in 32-bit, O += P V.  The four warps'
// partial results are merged through shared memory; a split that is not alone writes its
// unnormalised result and (max, sum) to the workspace, and a second small kernel merges the
// splits.  Unused MMA rows (fewer than 16 heads per kv head) cost nothing that matters: the
// kernel is bound by the cache's bytes.
//
// Compiled per head size: -DHOS_HEAD_DIM=N, N a multiple of 16 up to 256.
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_utils.cuh"

#ifndef HOS_HEAD_DIM
#define HOS_HEAD_DIM 64
#endif

namespace hos {

constexpr int HD = HOS_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16, at most 256");

constexpr int kTileBytes = kPageTokens * HD * 2;                    // one [64][HD] bf16 tile
constexpr int kStages = (2 * kTileBytes * 4 + 16 * HD * 2 <= 200 * 1024) ? 4 : 3;
constexpr int kQBytes = 16 * HD * 2;
constexpr int kDecodeSmem = kStages * 2 * kTileBytes + kQBytes + 64;
constexpr int kMaxHeadsPerCta = 16;

__device__ int g_decode_error = 0;     // set when a bounded wait gave up

struct DecodeArgs {
    const bf16* q;
    int q_stride;
    bf16* out;
    int out_stride;
    float* part_o;        // [N][n_heads][n_splits][HD]
    float* part_ml;       // [N][n_heads][n_splits][2]
    const int* token_pos;
    const int* token_seq;
    const int* seq_slot;
    PagedKV cache;
    int n_heads;
    int n_splits;
    float scale, cap;
    int window;
};

__global__ void __launch_bounds__(128, 1) attn_decode_kernel(DecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw);                     // kStages x (K tile, V tile)
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw + kStages * 2 * kTileBytes);  // [16][HD]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + kStages * 2 * kTileBytes + kQBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, n = blockIdx.z;
    const int group = a.n_heads / a.cache.n_kv_heads;
    const int chunks = (group + kMaxHeadsPerCta - 1) / kMaxHeadsPerCta;
    const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
    const int head0 = kvh * group + chunk * kMaxHeadsPerCta;                  // first query head of this CTA
    const int n_rows = min(kMaxHeadsPerCta, group - chunk * kMaxHeadsPerCta);   // real rows of the tile

    const int seq = a.token_seq[n];
    if (seq < 0) {                         // padding row: a defined output, nothing read
        if (split == 0)
            for (int i = tid; i < n_rows * HD; i += 128)
                a.out[(size_t)n * a.out_stride + (size_t)head0 * HD + i] = __float2bfloat16(0.f);
        return;
    }
    const int pos = a.token_pos[n];
    const int lo = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
    const int lp_lo = lo / kPageTokens, lp_hi = pos / kPageTokens;
    const int n_lp = lp_hi - lp_lo + 1;
    const int per_split = (n_lp + a.n_splits - 1) / a.n_splits;
    const int lp_begin = lp_lo + split * per_split;
    const int lp_end = min(lp_begin + per_split, lp_hi + 1);
    const int n_tiles = max(0, lp_end - lp_begin);

    auto part_index = [&](int head) { return ((size_t)n * a.n_heads + head) * a.n_splits + split; };
    if (n_tiles == 0) {                    // more splits than pages: an empty share
        for (int i = tid; i < n_rows; i += 128) {
            a.part_ml[part_index(head0 + i) * 2 + 0] = -INFINITY;
            a.part_ml[part_index(head0 + i) * 2 + 1] = 0.f;
        }
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    // Q rows (zero beyond the real heads), permuted like the key tiles
    {
        const bf16* qp = a.q + (size_t)n * a.q_stride + (size_t)head0 * HD;
        constexpr int chunks_per_row = HD / 8;
        for (int i = tid; i < 16 * chunks_per_row; i += 128) {
            const int r = i / chunks_per_row, c = i % chunks_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n_rows) v = *reinterpret_cast<const uint4*>(qp + (size_t)r * HD + c * 8);
            *reinterpret_cast<uint4*>(q_s + tile_chunk_offset<HD>(r, c)) = v;
        }
    }
    __syncthreads();

    const int slot = a.seq_slot[seq];
    const int* table = a.cache.page_table + (size_t)slot * a.cache.table_stride;
    const bf16* k_pages = reinterpret_cast<const bf16*>(a.cache.k_pages);
    const bf16* v_pages = reinterpret_cast<const bf16*>(a.cache.v_pages);
    auto issue = [&](int tile) {           // one thread: bring tile `tile` of this share on chip
        const int s = tile % kStages;
        const int page = table[kv_table_entry(a.cache, lp_begin + tile)];
        const size_t off = kv_tile_offset(a.cache, page, kvh);
        bf16* dst = stage_base + (size_t)s * 2 * (kTileBytes / 2);
        mbar_expect_tx(&full[s], 2 * kTileBytes);
        bulk_g2s(dst, k_pages + off, kTileBytes, &full[s]);
        bulk_g2s(dst + kTileBytes / 2, v_pages + off, kTileBytes, &full[s]);
    };
    if (tid == 0)
        for (int t = 0; t < min(kStages, n_tiles); ++t) issue(t);

    const int g = lane >> 2, t4 = lane & 3;
    const float inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const uint32_t q_base = smem_u32(q_s);
    bool gave_up = false;
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int s = tile % kStages;
        if (!mbar_wait(&full[s], (tile / kStages) & 1)) { gave_up = true; break; }
        const bf16* k_s = stage_base + (size_t)s * 2 * (kTileBytes / 2);
        const bf16* v_s = k_s + kTileBytes / 2;
        const uint32_t k_base = smem_u32(k_s), v_base = smem_u32(v_s);

        // ---- S = Q K^T for this warp's 16 keys ----
        float sc[2][4] = {};
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t qa[4], kb[4];
            {
                const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int ch = kk * 2 + (lane >> 4);
                ldmatrix_x4(qa, q_base + 2 * tile_chunk_offset<HD>(row, ch));
            }
            {
                const int row = warp * 16 + (lane & 7) + (lane >> 4) * 8;
                const int ch = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(kb, k_base + 2 * tile_chunk_offset<HD>(row, ch));
            }
            mma_bf16(sc[0], qa, kb[0], kb[1]);
            mma_bf16(sc[1], qa, kb[2], kb[3]);
        }
        // ---- scale, soft-cap, mask, running softmax ----
        const int key0 = (lp_begin + tile) * kPageTokens + warp * 16;
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = key0 + nt * 8 + 2 * t4 + (i & 1);
                float v = softcap_fast(sc[nt][i] * a.scale, a.cap, inv_cap);
                v = (key >= lo && key <= pos) ? v : -INFINITY;
                sc[nt][i] = v;
                m_new[i >> 1] = fmaxf(m_new[i >> 1], v);
            }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
            m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            m_use[r] = m_new[r] == -INFINITY ? 0.f : m_new[r];
            corr[r] = __expf(m_run[r] - m_use[r]);
            m_run[r] = m_new[r];
            l_run[r] *= corr[r];
        }
        uint32_t pa[4];
        {
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    p[nt][i] = __expf(sc[nt][i] - m_use[i >> 1]);
                    l_run[i >> 1] += p[nt][i];
                }
            pa[0] = pack_bf16(p[0][0], p[0][1]);
            pa[1] = pack_bf16(p[0][2], p[0][3]);
            pa[2] = pack_bf16(p[1][0], p[1][1]);
            pa[3] = pack_bf16(p[1][2], p[1][3]);
        }
        // ---- O = O * corr + P V ----
#pragma unroll
        for (int dd = 0; dd < HD / 16; ++dd) {
            uint32_t vb[4];
            const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int ch = dd * 2 + (lane >> 4);
            ldmatrix_x4_trans(vb, v_base + 2 * tile_chunk_offset<HD>(row, ch));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float* acc = o[dd * 2 + h];
                acc[0] *= corr[0]; acc[1] *= corr[0]; acc[2] *= corr[1]; acc[3] *= corr[1];
            }
            mma_bf16(o[dd * 2], pa, vb[0], vb[1]);
            mma_bf16(o[dd * 2 + 1], pa, vb[2], vb[3]);
        }
        __syncthreads();                   // every warp is done with stage s
        if (tid == 0 && tile + kStages < n_tiles) issue(tile + kStages);
    }
    if (gave_up) {
        if (lane == 0) atomicExch(&g_decode_error, 1);
        return;
    }
    // ---- merge the four warps (each saw other keys) through shared memory ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    __syncthreads();
    float* mo = reinterpret_cast<float*>(smem_raw);            // [4 warps][16 rows][HD]
    float* mml = mo + 4 * 16 * HD;                              // [4][16][2]
    static_assert(4 * 16 * HD * 4 + 4 * 16 * 2 * 4 <= kStages * 2 * kTileBytes, "merge area fits the stages");
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        float* b0 = mo + ((size_t)warp * 16 + g) * HD + i * 8 + 2 * t4;
        float* b1 = mo + ((size_t)warp * 16 + g + 8) * HD + i * 8 + 2 * t4;
        b0[0] = o[i][0]; b0[1] = o[i][1];
        b1[0] = o[i][2]; b1[1] = o[i][3];
    }
    if (t4 == 0) {
        mml[(warp * 16 + g) * 2 + 0] = m_run[0];
        mml[(warp * 16 + g) * 2 + 1] = l_run[0];
        mml[(warp * 16 + g + 8) * 2 + 0] = m_run[1];
        mml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    for (int idx = tid; idx < n_rows * HD; idx += 128) {
        const int r = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = mml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : __expf(mw - M);
            L += mml[(w * 16 + r) * 2 + 1] * f;
            acc += mo[((size_t)w * 16 + r) * HD + d] * f;
        }
        const int head = head0 + r;
        if (a.n_splits == 1) {
            a.out[(size_t)n * a.out_stride + (size_t)head * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
        } else {
            a.part_o[part_index(head) * HD + d] = acc;
            if (d == 0) {
                a.part_ml[part_index(head) * 2 + 0] = M;
                a.part_ml[part_index(head) * 2 + 1] = L;
            }
        }
    }
}

// Merge the splits of one (token, head): out = sum_s O_s e^{M_s - M} / sum_s L_s e^{M_s - M}.
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           bf16* __restrict__ out, int out_stride,
                                           const int* __restrict__ token_seq, int n_heads, int n_splits) {
    const int n = blockIdx.x / n_heads, head = blockIdx.x % n_heads;
    if (token_seq[n] < 0) return;          // the padding row was written by the first kernel
    const size_t base = ((size_t)n * n_heads + head) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(base + s) * 2];
        if (ms != -INFINITY) L += part_ml[(base + s) * 2 + 1] * __expf(ms - M);
    }
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(base + s) * 2];
            if (ms != -INFINITY) acc += part_o[(base + s) * HD + d] * __expf(ms - M);
        }
        out[(size_t)n * out_stride + (size_t)head * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
    }
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }
extern "C" int hos_attn_head_dim() { return HD; }

// Floats of workspace the kernel needs for these sizes (0 when one split is enough).
extern "C" long long hos_attn_decode_workspace(int n_tokens, int n_heads, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (HD + 2);
}

// 1 if an earlier launch gave up a bounded wait (and clears the flag).
extern "C" int hos_attn_decode_error() {
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_decode_error, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_decode_error, &zero, sizeof(int));
    return v;
}

extern "C" int hos_attn_decode(const void* q, int q_stride, void* out, int out_stride, float* workspace,
                               const int* token_pos, const int* token_seq, const int* seq_slot,
                               void* k_pages, void* v_pages, const int* page_table, int table_stride,
                               int ring_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                               float scale, float cap, int window, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim != HD) HOS_REFUSE("attn_decode: built for head_dim %d, asked for %d", HD, head_dim);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_decode: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (n_splits < 1 || n_splits > 65535) HOS_REFUSE("attn_decode: %d splits", n_splits);
    if (n_tokens > 65535) HOS_REFUSE("attn_decode: %d tokens are more than one launch takes", n_tokens);
    if (n_splits > 1 && workspace == nullptr) HOS_REFUSE("attn_decode: splits need a workspace");
    if ((q_stride % 8) != 0 || ((uintptr_t)q % 16) != 0)
        HOS_REFUSE("attn_decode: query rows must be 16-byte aligned");
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem);
        attr_set = true;
    }
    const int group = n_heads / n_kv_heads;
    const int chunks = (group + kMaxHeadsPerCta - 1) / kMaxHeadsPerCta;
    DecodeArgs a;
    a.q = (const bf16*)q; a.q_stride = q_stride;
    a.out = (bf16*)out; a.out_stride = out_stride;
    a.part_o = workspace;
    a.part_ml = workspace ? workspace + (size_t)n_tokens * n_heads * n_splits * HD : nullptr;
    a.token_pos = token_pos; a.token_seq = token_seq; a.seq_slot = seq_slot;
    a.cache = PagedKV{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim};
    a.n_heads = n_heads; a.n_splits = n_splits; a.scale = scale; a.cap = cap; a.window = window;
    dim3 grid(n_splits, n_kv_heads * chunks, n_tokens);
    attn_decode_kernel<<<grid, 128, kDecodeSmem, stream>>>(a);
    int rc = check_launch("attn_decode");
    if (rc) return rc;
    if (n_splits > 1) {
        attn_decode_combine_kernel<<<n_tokens * n_heads, HD >= 128 ? 128 : 64, 0, stream>>>(
            a.part_o, a.part_ml, a.out, out_stride, token_seq, n_heads, n_splits);
        rc = check_launch("attn_decode_combine");
    }
    return rc;
}
