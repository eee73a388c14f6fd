// Attention of single tokens over the paged cache (decoding), bfloat16, split over the keys.
//
// A work item is one token, one kv head (with the up to 16 query heads that share it, stacked
// as the rows of one MMA tile) and one contiguous share of the sequence's pages.  The kernel
// is persistent: one CTA per SM walks over the items.  A page's [64][HD] key tile and value
// tile are contiguous in the cache, so the producer warp brings each on chip with a single
// bulk copy (TMA) counted on an mbarrier, running ahead of the math through a ring of stages
// and across item boundaries, so that the memory pipe does not drain while an item is
// finished.  Four consumer warps take 16 keys of a tile each: S = Q K^T (m16n8k16, bf16, 32-bit
// accumulators), scale, soft-cap, mask, running max/sum in 32-bit, O += P V.  The four warps'
// partial results are merged through shared memory.  The shares of a (token, kv head) are then
// merged in one of two ways.  When there are at most 16 of them and all of a launch's items run
// at once, the launch is made of clusters, one per (token, kv head): every CTA leaves its
// unnormalised result and (max, sum) in its own shared memory, the cluster meets at a barrier,
// and every CTA merges a slice of the columns, reading the others' results through distributed
// shared memory.  Otherwise a share writes its result to the workspace and takes a ticket; the
// CTA that takes the last ticket of a (token, kv head) merges the shares.  Unused MMA
// rows (fewer than 16 heads per kv head) cost nothing that matters: the kernel is bound by
// the cache's bytes.
//
// The kernel has a second way to cut the work (attn_decode_kernel<true>, asked for with 0 shares): not every
// (token, kv head) into the same number of shares, but the row of all pages of all (token, kv head) into one
// piece of equal length per CTA, wherever the borders fall (see EvenPlan).  That wins where equal shares would
// leave a round of SMs mostly empty, and where the sequences are of unequal lengths.
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
constexpr int kStageBytes = 2 * kTileBytes;                         // keys and values of one page
constexpr int kQBytes = 16 * HD * 2;
constexpr int kMaxHeadsPerCta = 16;
constexpr int kMaxStages = 8;
constexpr int kMaxSplits = 64;
constexpr int kSmemBudget = 226 * 1024;
constexpr int kConsumers = 128, kDecodeThreads = 160;
constexpr long long kWaitCycles = 1ll << 31;                        // about a second

__device__ int g_decode_error = 0;     // set when a bounded wait gave up
__device__ int* g_decode_error_host = nullptr;     // a word in pinned host memory, if the host gave one

__device__ __forceinline__ void record_give_up() {
    atomicExch(&g_decode_error, 1);
    int* w = g_decode_error_host;
    if (w != nullptr) {
        atomicExch_system(w, kGiveUpAttnDecode);
        __threadfence_system();
    }
}

struct DecodeArgs {
    const bf16* q;
    int q_stride;
    bf16* out;
    int out_stride;
    float* part_o;        // [N][n_heads][n_splits][HD]
    float* part_ml;       // [N][n_heads][n_splits][2]
    int* tickets;         // [N][n_kv_heads * chunks], zero between launches
    const int* token_pos;
    const int* token_seq;
    const int* seq_slot;
    const int* token_slot;    // seq_slot[token_seq[n]] for every token, or null: one dependent load less before the first copy
    PagedKV cache;
    int n_tokens, n_heads, n_splits;
    int stages, merge_rows;
    float scale, cap;
    int window;
    int max_new;          // most new tokens any sequence brings in this step: what lies below them is old
    int cluster_merge;    // 1: the shares of a (token, kv head) are the CTAs of one cluster and merge through shared memory
};

__device__ __forceinline__ bool wait_timed(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > kWaitCycles) return false;
    return true;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A 32-bit float at the same shared-memory address in CTA `rank` of this cluster.
__device__ __forceinline__ float ld_cluster(const float* p, int rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// What an item is and which pages it covers: the same arithmetic on both sides of the pipe.
struct Item {
    int n, y, kvh, head0, n_rows;            // y: (kv head, chunk of 16 query heads) of the token
    int seq, pos, slot, lo, lp_begin, n_tiles;
    int part, n_parts, first_cta;            // which of the (token, y)'s shares this is; with even shares: the CTA of share 0
};
// everything but the share: the heads, the sequence, its slot and the lowest visible key
__device__ __forceinline__ void item_base(const DecodeArgs& a, Item& it, int n, int y, int group, int chunks) {
    it.n = n;
    it.y = y;
    it.kvh = y / chunks;
    const int chunk = y % chunks;
    it.head0 = it.kvh * group + chunk * kMaxHeadsPerCta;
    it.n_rows = min(kMaxHeadsPerCta, group - chunk * kMaxHeadsPerCta);
    // the three look-ups go out together; only the slot of a step that gives none waits for the sequence
    it.seq = a.token_seq[n];
    it.pos = a.token_pos[n];
    it.slot = a.token_slot != nullptr ? a.token_slot[n] : -1;
    it.lo = 0; it.lp_begin = 0; it.n_tiles = 0;
    it.part = 0; it.n_parts = 1; it.first_cta = 0;
    if (it.seq < 0) { it.pos = 0; return; }
    if (a.token_slot == nullptr) it.slot = a.seq_slot[it.seq];
    it.lo = a.window > 0 ? max(0, it.pos + 1 - a.window) : 0;
}
// Equal shares: every (token, y) is cut into n_splits shares of its own pages; item `index` is one share.
__device__ __forceinline__ Item make_item(const DecodeArgs& a, int index, int group, int chunks) {
    Item it;
    const int per_token = a.cache.n_kv_heads * chunks * a.n_splits;
    const int r = index % per_token;
    item_base(a, it, index / per_token, r / a.n_splits, group, chunks);
    it.part = r % a.n_splits;
    it.n_parts = a.n_splits;
    if (it.seq < 0) return it;
    const int lp_lo = it.lo / kPageTokens, lp_hi = it.pos / kPageTokens;
    const int n_lp = lp_hi - lp_lo + 1;
    const int per_split = (n_lp + a.n_splits - 1) / a.n_splits;
    it.lp_begin = lp_lo + it.part * per_split;
    const int lp_end = min(it.lp_begin + per_split, lp_hi + 1);
    it.n_tiles = max(0, lp_end - it.lp_begin);
    return it;
}

// Even shares: the pages of all (token, y) in one row (tokens in order, within a token y in order, within that
// the pages in order), and every CTA takes the same number of consecutive pages of that row, wherever the borders
// of the (token, y) fall.  With items of equal size a number of items that is no multiple of the SMs leaves SMs
// idle for a whole item's time (160 items on 148 SMs: twice the time of 148); cut like this, no CTA has more than
// one page more than another.  A (token, y) that lies in several CTAs is merged by the CTA that finishes last
// (tickets), from two places per CTA in the workspace: the share of a (token, y) that began in an earlier CTA is
// a CTA's first piece of work (place 0), the share of one that goes on in the next CTA its last (place 1).
struct EvenPlan {
    const int* pre;        // shared memory [n_tokens + 1]: pages of one y of the tokens before token n
    int per_token;         // (kv head, chunk) pairs per token
    int per_cta;           // pages per CTA
    long long total;       // pages in the row
};
struct EvenWalk {
    int n, y, off;         // the next piece: token, y, pages of that (token, y) already given out
    long long at, end;     // where this CTA stands in the row, and where it stops
};
__device__ __forceinline__ EvenWalk even_begin(const EvenPlan& e, int n_tokens) {
    EvenWalk w;
    w.at = (long long)blockIdx.x * e.per_cta;
    w.end = min(e.total, w.at + e.per_cta);
    w.n = 0; w.y = 0; w.off = 0;
    if (w.at >= w.end) return w;
    int lo = 0, hi = n_tokens - 1;              // the last token whose pages begin at or before `at` and that has pages
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((long long)e.pre[mid] * e.per_token <= w.at) lo = mid; else hi = mid - 1;
    }
    while (e.pre[lo + 1] == e.pre[lo]) --lo;    // (a token without pages begins where the next one does)
    const int pages = e.pre[lo + 1] - e.pre[lo];
    const long long rem = w.at - (long long)e.pre[lo] * e.per_token;
    w.n = lo;
    w.y = (int)(rem / pages);
    w.off = (int)(rem % pages);
    return w;
}
// The next piece of this CTA's walk: false when there is none.
__device__ __forceinline__ bool even_next(const DecodeArgs& a, const EvenPlan& e, EvenWalk& w, Item& it, int group, int chunks) {
    if (w.at >= w.end) return false;
    const int pages = e.pre[w.n + 1] - e.pre[w.n];
    const int take = (int)min((long long)(pages - w.off), w.end - w.at);
    item_base(a, it, w.n, w.y, group, chunks);
    it.lp_begin = it.lo / kPageTokens + w.off;
    it.n_tiles = take;
    const long long start = (long long)e.pre[w.n] * e.per_token + (long long)w.y * pages;
    it.first_cta = (int)(start / e.per_cta);
    it.n_parts = (int)((start + pages - 1) / e.per_cta) - it.first_cta + 1;
    it.part = (int)blockIdx.x - it.first_cta;
    w.at += take;
    w.off += take;
    if (w.off == pages) {
        w.off = 0;
        if (++w.y == e.per_token) {
            w.y = 0;
            do { ++w.n; } while (w.n < a.n_tokens && e.pre[w.n + 1] == e.pre[w.n]);
        }
    }
    return true;
}
constexpr int kEvenMaxTokens = 2048;   // rows of a step with even shares (their running sums live in shared memory)
constexpr int kEvenMaxParts = 32;      // a (token, y) lies in at most this many CTAs (the CTAs' shares grow if need be)

template <bool EVEN>
__global__ void __launch_bounds__(kDecodeThreads, 1) attn_decode_kernel(DecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int stages = a.stages;
    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw);                       // stages x (K tile, V tile)
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw + (size_t)stages * kStageBytes);  // [16][HD]
    float* mo = reinterpret_cast<float*>(smem_raw + (size_t)stages * kStageBytes + kQBytes);   // [4][merge_rows][HD]
    float* mml = mo + 4 * a.merge_rows * HD;                                    // [4][merge_rows][2]
    float* wm = mml + 4 * a.merge_rows * 2;                                     // [merge_rows][kMaxSplits] share weights
    float* wl = wm + a.merge_rows * kMaxSplits;                                 // [merge_rows][kMaxSplits]
    float* res = wl + a.merge_rows * kMaxSplits;                                // [merge_rows][HD + 2]: this share's result, for the cluster
    uint64_t* full = reinterpret_cast<uint64_t*>(res + a.merge_rows * (HD + 2));   // [stages]
    uint64_t* empty = full + kMaxStages;                                        // [stages]
    int* pre = reinterpret_cast<int*>(empty + kMaxStages);                      // even shares: [n_tokens + 1]
    __shared__ int last_flag;
    __shared__ int even_most;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = a.n_heads / a.cache.n_kv_heads;
    const int chunks = (group + kMaxHeadsPerCta - 1) / kMaxHeadsPerCta;
    const int total_items = EVEN ? 0 : a.n_tokens * a.cache.n_kv_heads * chunks * a.n_splits;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        mbar_fence_init();
        even_most = 1;
    }
    __syncthreads();
    EvenPlan plan{pre, a.cache.n_kv_heads * chunks, 1, 0};
    if (EVEN) {
        // pages per token (positions and sequences were written at the head of the step, long before this kernel),
        // their running sum, and the most pages of one token; padding rows have none
        int most = 0;
        for (int n = tid; n < a.n_tokens; n += kDecodeThreads) {
            int pages = 0;
            if (a.token_seq[n] >= 0) {
                const int pos = a.token_pos[n];
                const int lo = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
                pages = pos / kPageTokens - lo / kPageTokens + 1;
            }
            pre[n + 1] = pages;
            most = max(most, pages);
        }
        if (most > 1) atomicMax(&even_most, most);
        __syncthreads();
        if (warp == 0) {                       // running sum, 32 tokens at a time
            int carry = 0;
            for (int n0 = 0; n0 < a.n_tokens; n0 += 32) {
                const int n = n0 + lane;
                int v = n < a.n_tokens ? pre[n + 1] : 0;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int u = __shfl_up_sync(0xffffffffu, v, o);
                    if (lane >= o) v += u;
                }
                if (n < a.n_tokens) pre[n + 1] = carry + v;
                carry += __shfl_sync(0xffffffffu, v, 31);
            }
            if (lane == 0) pre[0] = 0;
        }
        __syncthreads();
        plan.total = (long long)pre[a.n_tokens] * plan.per_token;
        const long long even = (plan.total + gridDim.x - 1) / gridDim.x;
        const int least = (even_most + kEvenMaxParts - 2) / (kEvenMaxParts - 1);     // so that no (token, y) lies in too many CTAs
        plan.per_cta = (int)max(even, (long long)max(1, least));
    }
    pdl_launch_dependents();
    // This kernel is launched so that it may start while the projection before it still runs.  That
    // kernel writes q and the step's new keys and values, nothing else that is read here: the
    // producer may look up pages and fetch tiles that lie wholly below the step's new positions
    // before pdl_wait(); everything else comes after it.  (The slot and page tables were written
    // at least two kernels earlier.  In a ring the oldest tile of the window can share its page
    // with the newest positions: the rows that are being written are masked in that tile.)

    if (warp == 4) {
        // ---------------- producer: one thread feeds the ring, item after item ----------------
        if (lane == 0) {
            const bf16* k_pages = reinterpret_cast<const bf16*>(a.cache.k_pages);
            const bf16* v_pages = reinterpret_cast<const bf16*>(a.cache.v_pages);
            int t = 0;            // tiles issued so far by this CTA
            bool ok = true, waited = false;
            EvenWalk walk = even_begin(plan, a.n_tokens);
            for (int index = blockIdx.x; ok; index += gridDim.x) {
                Item it;
                if (EVEN) {
                    if (!even_next(a, plan, walk, it, group, chunks)) break;
                } else {
                    if (index >= total_items) break;
                    it = make_item(a, index, group, chunks);
                }
                if (it.n_tiles == 0) continue;
                const int* table = a.cache.page_table + (size_t)it.slot * a.cache.table_stride;
                for (int tile = 0; tile < it.n_tiles; ++tile, ++t) {
                    const int s = t % stages;
                    if (!waited && (t >= stages || (it.lp_begin + tile + 1) * kPageTokens > it.pos + 1 - a.max_new)) {
                        pdl_wait();
                        waited = true;
                    }
                    if (t >= stages && !wait_timed(&empty[s], ((t / stages) - 1) & 1)) { ok = false; break; }
                    const int page = table[kv_table_entry(a.cache, it.lp_begin + tile)];
                    const size_t off = kv_tile_offset(a.cache, page, it.kvh);
                    bf16* dst = stage_base + (size_t)s * (kStageBytes / 2);
                    mbar_expect_tx(&full[s], kStageBytes);
                    bulk_g2s(dst, k_pages + off, kTileBytes, &full[s]);
                    bulk_g2s(dst + kTileBytes / 2, v_pages + off, kTileBytes, &full[s]);
                }
            }
            if (!ok) record_give_up();
        }
        if (a.cluster_merge) {
            // one item per CTA; the whole cluster meets twice around the merge unless its token is padding
            __syncwarp();
            if (blockIdx.x < total_items && a.token_seq[blockIdx.x / (total_items / a.n_tokens)] >= 0) {
                cluster_barrier();
                cluster_barrier();
            }
        }
        return;
    }

    // ---------------- consumers: warps 0..3 ----------------
    pdl_wait();                   // q and the newest keys are complete from here on
    if (EVEN) {                   // padding rows are nobody's work here: a defined output for them
        for (int n = blockIdx.x; n < a.n_tokens; n += gridDim.x)
            if (pre[n + 1] == pre[n])
                for (int i = tid; i < a.n_heads * HD; i += kConsumers)
                    a.out[(size_t)n * a.out_stride + i] = __float2bfloat16(0.f);
    }
    const int g = lane >> 2, t4 = lane & 3;
    const float inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
    const uint32_t q_base = smem_u32(q_s);
    int t = 0;                    // tiles consumed so far by this CTA
    bool gave_up = false;

    EvenWalk walk = even_begin(plan, a.n_tokens);
    for (int index = blockIdx.x;; index += gridDim.x) {
        Item it;
        if (EVEN) {
            if (!even_next(a, plan, walk, it, group, chunks)) break;
        } else {
            if (index >= total_items) break;
            it = make_item(a, index, group, chunks);
        }
        const int n = it.n;
        const int mr = a.merge_rows;
        // Where share s of this (token, y) leaves row r of its result.  Equal shares: [token][head][share].  Even
        // shares: [CTA][place][row], place 1 for the share that begins the (token, y), place 0 for the others.
        auto part_row = [&](int r, int s) -> size_t {
            if (EVEN) return ((size_t)(it.first_cta + s) * 2 + (s == 0 ? 1 : 0)) * mr + r;
            return ((size_t)n * a.n_heads + it.head0 + r) * a.n_splits + s;
        };
        if (it.seq < 0) {                      // padding row: a defined output, nothing read
            if (it.part == 0)
                for (int i = tid; i < it.n_rows * HD; i += kConsumers)
                    a.out[(size_t)n * a.out_stride + (size_t)it.head0 * HD + i] = __float2bfloat16(0.f);
            continue;
        }
        // Q rows (zero beyond the real heads), permuted like the key tiles
        consumer_sync();                       // the last item's readers of q_s and of the merge area are done
        {
            const bf16* qp = a.q + (size_t)n * a.q_stride + (size_t)it.head0 * HD;
            constexpr int chunks_per_row = HD / 8;
            for (int i = tid; i < 16 * chunks_per_row; i += kConsumers) {
                const int r = i / chunks_per_row, c = i % chunks_per_row;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (r < it.n_rows) v = *reinterpret_cast<const uint4*>(qp + (size_t)r * HD + c * 8);
                *reinterpret_cast<uint4*>(q_s + tile_chunk_offset<HD>(r, c)) = v;
            }
        }
        consumer_sync();

        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        float o[HD / 8][4];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

        for (int tile = 0; tile < it.n_tiles; ++tile, ++t) {
            const int s = t % stages;
            if (!wait_timed(&full[s], (t / stages) & 1)) { gave_up = true; break; }      // (the whole CTA: the barrier is one)
            const bf16* k_s = stage_base + (size_t)s * (kStageBytes / 2);
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
            const int key0 = (it.lp_begin + tile) * kPageTokens + warp * 16;
            float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = key0 + nt * 8 + 2 * t4 + (i & 1);
                    float v = softcap_fast(sc[nt][i] * a.scale, a.cap, inv_cap);
                    v = (key >= it.lo && key <= it.pos) ? v : -INFINITY;
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
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);      // this warp is done with the stage
        }
        if (gave_up && !a.cluster_merge) break;      // in a cluster the others wait for this CTA at the barriers below

        // ---- merge the four warps (each saw other keys) through shared memory ----
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
            l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = g + 8 * h;
            if (row < it.n_rows) {
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) {
                    float* b = mo + ((size_t)warp * mr + row) * HD + i * 8 + 2 * t4;
                    b[0] = o[i][2 * h];
                    b[1] = o[i][2 * h + 1];
                }
                if (t4 == 0) {
                    mml[(warp * mr + row) * 2 + 0] = m_run[h];
                    mml[(warp * mr + row) * 2 + 1] = l_run[h];
                }
            }
        }
        consumer_sync();
        for (int idx = tid; idx < it.n_rows * HD; idx += kConsumers) {
            const int r = idx / HD, d = idx % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * mr + r) * 2]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = mml[(w * mr + r) * 2];
                const float f = mw == -INFINITY ? 0.f : __expf(mw - M);
                L += mml[(w * mr + r) * 2 + 1] * f;
                acc += mo[((size_t)w * mr + r) * HD + d] * f;
            }
            const int head = it.head0 + r;
            if (it.n_parts == 1) {
                a.out[(size_t)n * a.out_stride + (size_t)head * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
            } else if (!EVEN && a.cluster_merge) {
                res[r * (HD + 2) + d] = acc;
                if (d == 0) {
                    res[r * (HD + 2) + HD] = M;
                    res[r * (HD + 2) + HD + 1] = L;
                }
            } else {
                const size_t at = part_row(r, it.part);
                a.part_o[at * HD + d] = acc;
                if (d == 0) {
                    a.part_ml[at * 2 + 0] = M;
                    a.part_ml[at * 2 + 1] = L;
                }
            }
        }
        if (it.n_parts == 1) continue;
        if (!EVEN && a.cluster_merge) {
            // ---- the shares of this (token, kv head) are the CTAs of this cluster: every one of them merges a
            // slice of the columns, reading the others' results from their shared memory ----
            cluster_barrier();
            const int per_rank = (HD + a.n_splits - 1) / a.n_splits;
            const int d0 = it.part * per_rank, d1 = min(HD, d0 + per_rank);
            for (int idx = tid; idx < it.n_rows * (d1 - d0); idx += kConsumers) {
                const int r = idx / (d1 - d0), d = d0 + idx % (d1 - d0);
                float M = -INFINITY;
                for (int s = 0; s < a.n_splits; ++s) M = fmaxf(M, ld_cluster(res + r * (HD + 2) + HD, s));
                float L = 0.f, acc = 0.f;
                for (int s = 0; s < a.n_splits; ++s) {
                    const float ms = ld_cluster(res + r * (HD + 2) + HD, s);
                    const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
                    L += ld_cluster(res + r * (HD + 2) + HD + 1, s) * f;
                    if (f != 0.f) acc += ld_cluster(res + r * (HD + 2) + d, s) * f;
                }
                a.out[(size_t)n * a.out_stride + (size_t)(it.head0 + r) * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
            }
            cluster_barrier();                 // nobody leaves while its results are still being read
            if (gave_up) break;
            continue;
        }

        // ---- the share is written: take a ticket; the last share of (token, kv head) merges all ----
        __threadfence();
        consumer_sync();
        int* ticket = a.tickets + (size_t)n * a.cache.n_kv_heads * chunks + it.y;
        if (tid == 0) {
            last_flag = atomicAdd(ticket, 1) == it.n_parts - 1;
            if (last_flag) *ticket = 0;        // left at zero for the next launch
        }
        consumer_sync();
        if (!last_flag) continue;
        __threadfence();
        // weights of the shares, once per row: w_s = e^{M_s - M} / sum_s L_s e^{M_s - M} (0 for a share without keys)
        for (int i = tid; i < it.n_rows * it.n_parts; i += kConsumers) {
            const int r = i / it.n_parts, s = i % it.n_parts;
            const size_t at = part_row(r, s);
            wm[r * kMaxSplits + s] = __ldcg(&a.part_ml[at * 2]);
            wl[r * kMaxSplits + s] = __ldcg(&a.part_ml[at * 2 + 1]);
        }
        consumer_sync();
        if (tid < it.n_rows) {
            float M = -INFINITY, L = 0.f;
            for (int s = 0; s < it.n_parts; ++s) M = fmaxf(M, wm[tid * kMaxSplits + s]);
            for (int s = 0; s < it.n_parts; ++s) {
                const float ms = wm[tid * kMaxSplits + s];
                const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
                L += wl[tid * kMaxSplits + s] * f;
                wm[tid * kMaxSplits + s] = f;
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            for (int s = 0; s < it.n_parts; ++s) wm[tid * kMaxSplits + s] *= inv;
        }
        consumer_sync();
        for (int idx = tid; idx < it.n_rows * HD; idx += kConsumers) {
            const int r = idx / HD, d = idx % HD;
            const int head = it.head0 + r;
            const float* po = a.part_o + d;
            float acc = 0.f;
            int s = 0;
            for (; s + 8 <= it.n_parts; s += 8) {          // eight loads in flight; a share without keys wrote nothing
                float w[8], v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = wm[r * kMaxSplits + s + j];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = w[j] != 0.f ? __ldcg(po + part_row(r, s + j) * HD) : 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc += w[j] * v[j];
            }
            for (; s < it.n_parts; ++s) {
                const float w = wm[r * kMaxSplits + s];
                if (w != 0.f) acc += w * __ldcg(po + part_row(r, s) * HD);
            }
            a.out[(size_t)n * a.out_stride + (size_t)head * HD + d] = __float2bfloat16(acc);
        }
    }
    if (gave_up && lane == 0) record_give_up();
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }
extern "C" int hos_attn_head_dim() { return HD; }

// Whether few shares merge as a cluster (default) or through the workspace: HOS_ATTN_CLUSTER=0 or
// hos_attn_decode_cluster(0) keep the workspace.
static int& cluster_merge_state() {
    static int on = !(getenv("HOS_ATTN_CLUSTER") && getenv("HOS_ATTN_CLUSTER")[0] == '0');
    return on;
}
static bool cluster_merge_enabled() { return cluster_merge_state() != 0; }
extern "C" int hos_attn_decode_cluster(int on) {
    cluster_merge_state() = on ? 1 : 0;
    return 0;
}

// Floats of workspace the kernel needs for these sizes (0 when one share is enough), and the
// ints of tickets (which must be zero before the first launch; the kernel leaves them zero).
extern "C" long long hos_attn_decode_workspace(int n_tokens, int n_heads, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (HD + 2);
}
// The same for even shares: two places per CTA.
extern "C" long long hos_attn_decode_even_workspace(int n_heads, int n_kv_heads) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return 0;
    const int group = n_heads / n_kv_heads;
    return (long long)sm_count() * 2 * (group < kMaxHeadsPerCta ? group : kMaxHeadsPerCta) * (HD + 2);
}
extern "C" long long hos_attn_decode_tickets(int n_tokens, int n_heads, int n_kv_heads) {
    const int group = n_heads / n_kv_heads;
    return (long long)n_tokens * n_kv_heads * ((group + kMaxHeadsPerCta - 1) / kMaxHeadsPerCta);
}

// 1 if an earlier launch gave up a bounded wait (and clears the flag).
extern "C" int hos_attn_decode_error() {
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_decode_error, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_decode_error, &zero, sizeof(int));
    return v;
}

// The host's word for waits that ran out; null takes it away.
extern "C" int hos_attn_decode_set_error_word(int* word) {
    if (cudaMemcpyToSymbol(g_decode_error_host, &word, sizeof(word)) != cudaSuccess)
        HOS_REFUSE("attn_decode: cannot set the error word: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

// How many clusters of `size` CTAs with `smem` bytes each run on the GPU at once (0: such clusters cannot be had).
static int clusters_that_fit(int size, int smem) {
    static int known[17][2] = {};             // [cluster size]: (smem asked about, answer)
    if (size < 1 || size > 16) return 0;
    if (known[size][0] == smem) return known[size][1];
    static bool wide = false;
    if (size > 8 && !wide) {
        wide = cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        cudaGetLastError();
    }
    static int attr_smem = 0;
    if (smem > attr_smem &&
        cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess)
        attr_smem = smem;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)size);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = size; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if ((size > 8 && !wide) || cudaOccupancyMaxActiveClusters(&n, attn_decode_kernel<false>, &cfg) != cudaSuccess) n = 0;
    cudaGetLastError();
    known[size][0] = smem;
    known[size][1] = n;
    return n;
}
static int decode_smem(int group, int* stages_out, int even_tokens = 0) {
    const int merge_rows = group < kMaxHeadsPerCta ? group : kMaxHeadsPerCta;
    const int fixed = kQBytes + 5 * merge_rows * (HD + 2) * 4 + 2 * merge_rows * kMaxSplits * 4 + 2 * kMaxStages * 8 + 128 +
                      (even_tokens > 0 ? ((even_tokens + 1) * 4 + 15) / 16 * 16 : 0);
    int stages = (kSmemBudget - fixed) / kStageBytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages_out) *stages_out = stages;
    return stages * kStageBytes + fixed;
}
// Clusters of n_splits CTAs of this kernel that run at once for these heads (0: none): what the choice of the
// number of shares needs to know about the cluster merge.
extern "C" int hos_attn_decode_clusters(int n_heads, int n_kv_heads, int n_splits) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_splits < 2 || n_splits > 16) return 0;
    int stages = 0;
    const int smem = decode_smem(n_heads / n_kv_heads, &stages);
    return stages < 2 ? 0 : clusters_that_fit(n_splits, smem);
}

extern "C" int hos_attn_decode(const void* q, int q_stride, void* out, int out_stride, float* workspace,
                               int* tickets, const int* token_pos, const int* token_seq, const int* seq_slot,
                               const int* token_slot, void* k_pages, void* v_pages, const int* page_table, int table_stride,
                               int ring_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                               float scale, float cap, int window, int n_splits, int max_new, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (max_new < 1) HOS_REFUSE("attn_decode: max_new %d (the most new tokens of a sequence in this step) must be at least 1", max_new);
    if (head_dim != HD) HOS_REFUSE("attn_decode: built for head_dim %d, asked for %d", HD, head_dim);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_decode: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    const bool even = n_splits == 0;            // 0: even shares, every CTA the same number of pages
    if (n_splits < 0 || n_splits > kMaxSplits) HOS_REFUSE("attn_decode: %d splits (0: even shares, 1..%d)", n_splits, kMaxSplits);
    if (n_splits != 1 && (workspace == nullptr || tickets == nullptr))
        HOS_REFUSE("attn_decode: splits need a workspace and tickets");
    if (even && n_tokens > kEvenMaxTokens) HOS_REFUSE("attn_decode: even shares take up to %d rows, not %d", kEvenMaxTokens, n_tokens);
    if ((q_stride % 8) != 0 || ((uintptr_t)q % 16) != 0)
        HOS_REFUSE("attn_decode: query rows must be 16-byte aligned");
    const int group = n_heads / n_kv_heads;
    const int chunks = (group + kMaxHeadsPerCta - 1) / kMaxHeadsPerCta;
    const long long items = (long long)n_tokens * n_kv_heads * chunks * (even ? 1 : n_splits);
    if (items > (1ll << 30)) HOS_REFUSE("attn_decode: too many work items");
    DecodeArgs a;
    a.merge_rows = group < kMaxHeadsPerCta ? group : kMaxHeadsPerCta;
    int stages = 0;
    const int smem = decode_smem(group, &stages, even ? n_tokens : 0);
    if (stages < 2) HOS_REFUSE("attn_decode: shared memory holds fewer than two stages for head_dim %d", HD);
    a.stages = stages;
    static int attr_smem[2] = {0, 0};
    if (smem > attr_smem[even]) {
        const cudaError_t e = even
            ? cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
            : cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) HOS_REFUSE("attn_decode: cannot get %d bytes of shared memory", smem);
        attr_smem[even] = smem;
    }
    a.q = (const bf16*)q; a.q_stride = q_stride;
    a.out = (bf16*)out; a.out_stride = out_stride;
    a.part_o = workspace;
    a.part_ml = workspace ? workspace + (even ? (size_t)sm_count() * 2 * a.merge_rows : (size_t)n_tokens * n_heads * n_splits) * HD : nullptr;
    a.tickets = tickets;
    a.token_pos = token_pos; a.token_seq = token_seq; a.seq_slot = seq_slot; a.token_slot = token_slot;
    a.cache = PagedKV{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim};
    a.n_tokens = n_tokens; a.n_heads = n_heads; a.n_splits = n_splits;
    a.scale = scale; a.cap = cap; a.window = window; a.max_new = max_new;
    a.cluster_merge = 0;
    // Few items (one wave): the shares of a (token, kv head) run as one cluster and merge through shared memory
    // instead of through a workspace, a ticket and a last arrival; only if all the clusters fit on the GPU at once.
    if (n_splits > 1 && n_splits <= 16 && items <= sm_count() && cluster_merge_enabled()) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)items);
        cfg.blockDim = dim3(kDecodeThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = n_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        const int fit = clusters_that_fit(n_splits, smem);
        if ((long long)fit * n_splits >= items) {
            a.cluster_merge = 1;
            cfg.numAttrs = 2;
            cudaLaunchKernelEx(&cfg, attn_decode_kernel<false>, a);
            return check_launch("attn_decode (clusters)");
        }
    }
    if (even) {
        launch_ahead(true, attn_decode_kernel<true>, dim3(sm_count()), dim3(kDecodeThreads), smem, stream, a);
        return check_launch("attn_decode (even shares)");
    }
    const int grid = items < sm_count() ? (int)items : sm_count();
    launch_ahead(true, attn_decode_kernel<false>, dim3(grid), dim3(kDecodeThreads), smem, stream, a);
    return check_launch("attn_decode");
}

// ---- the entry point that allocates nothing (see attn_decode_noalloc.h) -----------------------
#include "attn_decode_noalloc.h"

namespace hos {
// Partial results of the shares, then the counters.  In host code this name is only a handle
// for cudaGetSymbolAddress: the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HOS_NOALLOC_SCRATCH_BYTES + HOS_NOALLOC_TICKETS * sizeof(int)];
constexpr int kMaxDevices = 64;
static void* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace hos

extern "C" int hos_attn_decode_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                       const int* token_pos, const int* token_seq, const int* seq_slot,
                                       void* k_pages, void* v_pages, const int* page_table, int table_stride,
                                       int ring_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                       float scale, float cap, int window, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_decode_noalloc: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (n_splits < 1) HOS_REFUSE("attn_decode_noalloc: %d splits", n_splits);
    const long long floats = hos_attn_decode_workspace(n_tokens, n_heads, n_splits);
    const long long pairs = hos_attn_decode_tickets(n_tokens, n_heads, n_kv_heads);
    if (floats * (long long)sizeof(float) > (long long)HOS_NOALLOC_SCRATCH_BYTES)
        HOS_REFUSE("attn_decode_noalloc: the partial results of %d tokens x %d heads x %d splits need %lld bytes, "
                   "the built-in scratch holds %u: use fewer splits or tokens, or hos_attn_decode with a workspace",
                   n_tokens, n_heads, n_splits, floats * (long long)sizeof(float), HOS_NOALLOC_SCRATCH_BYTES);
    if (pairs > HOS_NOALLOC_TICKETS)
        HOS_REFUSE("attn_decode_noalloc: %lld (token, kv head) pairs, the built-in counters hold %d", pairs,
                   HOS_NOALLOC_TICKETS);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        HOS_REFUSE("attn_decode_noalloc: cannot tell the current device");
    if (g_noalloc_ptr[dev] == nullptr) {       // once per device, with that device current
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            HOS_REFUSE("attn_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_noalloc_ptr[dev] = p;
    }
    unsigned char* base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
    float* workspace = reinterpret_cast<float*>(base);
    int* tickets = reinterpret_cast<int*>(base + HOS_NOALLOC_SCRATCH_BYTES);
    if (n_splits > 1) {                        // the counters must start at zero whatever the last call left
        cudaError_t e = cudaMemsetAsync(tickets, 0, (size_t)pairs * sizeof(int), stream);
        if (e != cudaSuccess) HOS_REFUSE("attn_decode_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
    }
    return hos_attn_decode(q, q_stride, out, out_stride, workspace, tickets, token_pos, token_seq, seq_slot, nullptr, k_pages,
                           v_pages, page_table, table_stride, ring_pages, n_tokens, n_heads, n_kv_heads, head_dim,
                           scale, cap, window, n_splits, /*max_new: nothing is fetched ahead*/ 1 << 30, stream);
}
