// Attention of many tokens per sequence, bfloat16, flash style, in two forms.
//
// Whole prompts that start at position 0: queries, keys and values are the rows of this
// step's own fused projection output, packed sequence after sequence (nothing is read from
// the cache).  Sequences that go on by many tokens (a prompt fed in pieces, a second turn):
// queries are the step's rows, keys and values are read from the paged cache, which holds
// the step's own keys already; a key tile is a page (or half of one), copied as it lies.
//
// One CTA (4 warps) takes 64
// consecutive queries of one sequence and one query head; key/value tiles of 64 rows (32 for
// head sizes above 128, where two CTAs then share an SM) stream
// through a two-stage cp.async pipeline into XOR-permuted shared memory.  Per tile each warp
// computes S = Q K^T for its 16 queries (m16n8k16 bf16, 32-bit accumulators), scales,
// soft-caps, masks (causal, and the window's lower edge), keeps a running max and sum in
// 32-bit, and accumulates O += P V.  Tiles wholly outside the window are skipped.
//
// Compiled per head size: -DHOS_HEAD_DIM=N, N a multiple of 16 up to 256.
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_utils.cuh"

#ifndef HOS_HEAD_DIM
#define HOS_HEAD_DIM 64
#endif

namespace hos {

constexpr int PHD = HOS_HEAD_DIM;
static_assert(PHD % 16 == 0 && PHD >= 16 && PHD <= 256, "head_dim must be a multiple of 16, at most 256");
constexpr int BQ = 64;
// keys per tile: 32 for the largest heads, so that two CTAs fit an SM's shared memory and registers
constexpr int BKV = PHD > 128 ? 32 : 64;
constexpr int KB = BKV / 16;                                  // blocks of 16 keys per tile
constexpr int kPrefillSmem = (BQ + 4 * BKV) * PHD * 2;        // Q + 2 stages x (K, V)

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const int sz = valid ? 16 : 0;                             // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(sz)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Copy `rows` x PHD bf16 from global rows (stride in elements) into a permuted smem tile;
// rows at or beyond `valid_rows` are zero-filled.
__device__ __forceinline__ void load_tile(bf16* tile, const bf16* src, int stride, int rows, int valid_rows) {
    constexpr int cpr = PHD / 8;
    for (int i = threadIdx.x; i < rows * cpr; i += 128) {
        const int r = i / cpr, c = i % cpr;
        const bool ok = r < valid_rows;
        cp_async_16(tile + tile_chunk_offset<PHD>(r, c), src + (size_t)(ok ? r : 0) * stride + c * 8, ok);
    }
}

// A tile of `rows` keys (or values) that lies contiguous and permuted in the cache: copied as it is.
__device__ __forceinline__ void load_tile_verbatim(bf16* tile, const bf16* src, int rows) {
    for (int i = threadIdx.x; i < rows * (PHD / 8); i += 128) cp_async_16(tile + i * 8, src + i * 8, true);
}

// PAGED = false: sequences from position 0, keys and values in rows k, v (stride kv_stride).
// PAGED = true: the rows of sequence s are cu_seqlens[s] - row_base .. of q and out, the first of
// them at position token_pos[that row]; keys and values come from `cache` through the page table
// row of seq_slot[s].
template <bool PAGED>
__global__ void __launch_bounds__(128, PHD > 128 ? 2 : 1)
attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k,
                    const bf16* __restrict__ v, int kv_stride, bf16* __restrict__ out, int out_stride,
                    const int* __restrict__ cu_seqlens, int n_seqs, int n_heads, int n_kv_heads,
                    float scale, float cap, int window, int row_base, const int* __restrict__ token_pos,
                    const int* __restrict__ seq_slot, PagedKV cache) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);
    bf16* kv_s = q_s + BQ * PHD;                               // stage s: K at 2s, V at 2s+1 (tiles of BKV*PHD)

    // which sequence and which block of 64 queries
    int seq = 0, tile_in_seq = blockIdx.x, row0 = 0, len = 0;
    for (; seq < n_seqs; ++seq) {
        row0 = cu_seqlens[seq] - row_base;
        len = cu_seqlens[seq + 1] - row_base - row0;
        const int nt = (len + BQ - 1) / BQ;
        if (tile_in_seq < nt) break;
        tile_in_seq -= nt;
    }
    if (seq >= n_seqs) return;
    const int head = blockIdx.y, kvh = head / (n_heads / n_kv_heads);
    const int q0 = tile_in_seq * BQ;                           // first query row of this CTA within its sequence
    const int q_rows = min(BQ, len - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int p0 = q0 + (PAGED ? token_pos[row0] : 0);         // and its position

    const int last_q = p0 + q_rows - 1;
    const int first_key = window > 0 ? max(0, p0 + 1 - window) : 0;
    const int kt_lo = first_key / BKV, kt_hi = last_q / BKV;
    const int n_kt = kt_hi - kt_lo + 1;

    const bf16* kbase = PAGED ? reinterpret_cast<const bf16*>(cache.k_pages) : k + (size_t)row0 * kv_stride + (size_t)kvh * PHD;
    const bf16* vbase = PAGED ? reinterpret_cast<const bf16*>(cache.v_pages) : v + (size_t)row0 * kv_stride + (size_t)kvh * PHD;
    const int* table = PAGED ? cache.page_table + (size_t)seq_slot[seq] * cache.table_stride : nullptr;
    load_tile(q_s, q + (size_t)(row0 + q0) * q_stride + (size_t)head * PHD, q_stride, BQ, q_rows);
    auto load_kv = [&](int kt, int stage) {
        const int key0 = kt * BKV;
        bf16* ks = kv_s + (size_t)(2 * stage) * BKV * PHD;
        bf16* vs = kv_s + (size_t)(2 * stage + 1) * BKV * PHD;
        if (PAGED) {
            // rows key0 % 64 .. of the page's tile: contiguous, and permuted by (row & 7) as the tile in
            // shared memory is (BKV is a multiple of 8).  Rows that no token has written yet hold zeros
            // or older keys: the causal mask and the window's lower edge leave them out.
            const int page = table[kv_table_entry(cache, key0 / kPageTokens)];
            const size_t off = kv_tile_offset(cache, page, kvh) + (size_t)(key0 % kPageTokens) * PHD;
            load_tile_verbatim(ks, kbase + off, BKV);
            load_tile_verbatim(vs, vbase + off, BKV);
        } else {
            load_tile(ks, kbase + (size_t)key0 * kv_stride, kv_stride, BKV, len - key0);
            load_tile(vs, vbase + (size_t)key0 * kv_stride, kv_stride, BKV, len - key0);
        }
    };
    load_kv(kt_lo, 0);
    cp_async_commit();

    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[PHD / 8][4];
#pragma unroll
    for (int i = 0; i < PHD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const uint32_t q_base = smem_u32(q_s);
    const int qpos[2] = {p0 + warp * 16 + g, p0 + warp * 16 + g + 8};

    for (int it = 0; it < n_kt; ++it) {
        const int stage = it & 1;
        if (it + 1 < n_kt) load_kv(kt_lo + it + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t k_base = smem_u32(kv_s + (size_t)(2 * stage) * BKV * PHD);
        const uint32_t v_base = smem_u32(kv_s + (size_t)(2 * stage + 1) * BKV * PHD);
        const int key0 = (kt_lo + it) * BKV;

        float sc[2 * KB][4];
#pragma unroll
        for (int i = 0; i < 2 * KB; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < PHD / 16; ++kk) {
            uint32_t qa[4];
            {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(qa, q_base + 2 * tile_chunk_offset<PHD>(row, kk * 2 + (lane >> 4)));
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                uint32_t b[4];
                const int row = kb * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(b, k_base + 2 * tile_chunk_offset<PHD>(row, kk * 2 + ((lane >> 3) & 1)));
                mma_bf16(sc[kb * 2], qa, b[0], b[1]);
                mma_bf16(sc[kb * 2 + 1], qa, b[2], b[3]);
            }
        }
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < 2 * KB; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = key0 + nt * 8 + 2 * t4 + (i & 1);
                const int qp = qpos[i >> 1];
                float s = softcap_fast(sc[nt][i] * scale, cap, inv_cap);
                const bool vis = key <= qp && (window <= 0 || key > qp - window);
                s = vis ? s : -INFINITY;
                sc[nt][i] = s;
                m_new[i >> 1] = fmaxf(m_new[i >> 1], s);
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
#pragma unroll
        for (int i = 0; i < PHD / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            uint32_t pa[4];
            {
                float p[2][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        p[h][i] = __expf(sc[kb * 2 + h][i] - m_use[i >> 1]);
                        l_run[i >> 1] += p[h][i];
                    }
                pa[0] = pack_bf16(p[0][0], p[0][1]);
                pa[1] = pack_bf16(p[0][2], p[0][3]);
                pa[2] = pack_bf16(p[1][0], p[1][1]);
                pa[3] = pack_bf16(p[1][2], p[1][3]);
            }
#pragma unroll
            for (int dd = 0; dd < PHD / 16; ++dd) {
                uint32_t vb[4];
                const int row = kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(vb, v_base + 2 * tile_chunk_offset<PHD>(row, dd * 2 + (lane >> 4)));
                mma_bf16(o[dd * 2], pa, vb[0], vb[1]);
                mma_bf16(o[dd * 2 + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();                   // the stage may be overwritten by the next iteration's loads
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = warp * 16 + g + r * 8;
        if (qi >= q_rows) continue;
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
        bf16* op = out + (size_t)(row0 + q0 + qi) * out_stride + (size_t)head * PHD;
#pragma unroll
        for (int i = 0; i < PHD / 8; ++i)
            *reinterpret_cast<uint32_t*>(op + i * 8 + 2 * t4) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
}

}  // namespace hos

using namespace hos;

// Sequences occupy rows cu_seqlens[s] .. cu_seqlens[s+1]-1, each from position 0; n_q_tiles is
// the sum over sequences of ceil(len / 64).  Rows beyond cu_seqlens[n_seqs] (padding) are not
// touched.
extern "C" int hos_attn_prefill(const void* q, int q_stride, const void* k, const void* v, int kv_stride,
                                void* out, int out_stride, const int* cu_seqlens, int n_seqs, int n_q_tiles,
                                int n_heads, int n_kv_heads, int head_dim, float scale, float cap, int window,
                                cudaStream_t stream) {
    if (n_q_tiles <= 0 || n_seqs <= 0) return 0;
    if (head_dim != PHD) HOS_REFUSE("attn_prefill: built for head_dim %d, asked for %d", PHD, head_dim);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_prefill: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (n_heads > 65535) HOS_REFUSE("attn_prefill: %d heads are more than one launch takes", n_heads);
    if ((q_stride % 8) || (kv_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)k % 16) ||
        ((uintptr_t)v % 16) || ((uintptr_t)out % 4))
        HOS_REFUSE("attn_prefill: rows must be 16-byte aligned");
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem);
        attr_set = true;
    }
    dim3 grid(n_q_tiles, n_heads);
    launch_pdl(attn_prefill_kernel<false>, dim3(grid), dim3(128), kPrefillSmem, stream,
        (const bf16*)q, q_stride, (const bf16*)k, (const bf16*)v, kv_stride, (bf16*)out, out_stride, cu_seqlens,
        n_seqs, n_heads, n_kv_heads, scale, cap, window, 0, (const int*)nullptr, (const int*)nullptr, PagedKV{});
    return check_launch("attn_prefill");
}

// Sequences that go on by many tokens, over the paged cache (which holds the step's keys already).
// Sequence s of the n_seqs has the rows cu_seqlens[s] - row_base .. cu_seqlens[s + 1] - row_base - 1 of q and
// out, at the positions token_pos[row] (consecutive within a sequence), and the page table row seq_slot[s];
// n_q_tiles is at least the sum over sequences of ceil(rows / 64).
extern "C" int hos_attn_chunk(const void* q, int q_stride, void* out, int out_stride, const int* cu_seqlens,
                              int row_base, const int* token_pos, const int* seq_slot, int n_seqs, int n_q_tiles,
                              void* k_pages, void* v_pages, const int* page_table, int table_stride, int ring_pages,
                              int n_heads, int n_kv_heads, int head_dim, float scale, float cap, int window,
                              cudaStream_t stream) {
    if (n_q_tiles <= 0 || n_seqs <= 0) return 0;
    if (head_dim != PHD) HOS_REFUSE("attn_chunk: built for head_dim %d, asked for %d", PHD, head_dim);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_chunk: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (n_heads > 65535) HOS_REFUSE("attn_chunk: %d heads are more than one launch takes", n_heads);
    if ((q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)k_pages % 16) ||
        ((uintptr_t)v_pages % 16) || ((uintptr_t)out % 4))
        HOS_REFUSE("attn_chunk: rows and pages must be 16-byte aligned");
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem);
        attr_set = true;
    }
    dim3 grid(n_q_tiles, n_heads);
    launch_pdl(attn_prefill_kernel<true>, dim3(grid), dim3(128), kPrefillSmem, stream,
        (const bf16*)q, q_stride, (const bf16*)nullptr, (const bf16*)nullptr, 0, (bf16*)out, out_stride, cu_seqlens,
        n_seqs, n_heads, n_kv_heads, scale, cap, window, row_base, token_pos, seq_slot,
        PagedKV{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim});
    return check_launch("attn_chunk");
}
