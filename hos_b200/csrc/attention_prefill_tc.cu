// Attention of whole prompts from position 0 on the 5th-generation tensor cores (head sizes
// 64, 128 and 256), bfloat16.
//
// One CTA takes 128 consecutive queries of one sequence and one query head and walks over
// key tiles of 64.  Queries, keys and values are rows of the step's fused projection output;
// TMA brings [rows x 64] column blocks of them into shared memory with the 128-byte swizzle.
// Per key tile:  S = Q K^T  (tcgen05.mma, M=128, N=64, K=head_dim; accumulator in tensor
// memory, two buffers so that the next tile's product runs under this tile's softmax);
// the softmax warps read S back (a thread's registers hold a run of one query row: no
// shuffles), scale, soft-cap, mask, exponentiate and write P as bfloat16 into shared memory in
// the K-major swizzled layout;  O += P V  (tcgen05.mma, M=128,
// N=head_dim, K=64, V used as it lies in memory: an MN-major operand), O staying in tensor
// memory for the whole walk.  The running maximum is only raised when a tile's maximum
// exceeds it by more than 8 (probabilities up to e^8 are harmless in 32-bit sums and
// bfloat16 P), so O is rescaled rarely; when it is, the thread reads its O row from tensor
// memory, scales it and writes it back.  At the end each thread divides its row by its sum
// and stores it.  Warp roles: 0 TMA, 1 MMA issue and tensor-memory allocation, 2-9 softmax,
// correction and epilogue: two threads per query row, each with 32 of a tile's 64 keys (warps w
// and w+4 share a quarter of the tensor-memory lanes), exchanging the row's maximum through
// shared memory.  P has two buffers, so the softmax of a tile does not wait for the P.V product
// of the tile before.  The soft-cap uses tanh.approx (relative error 2^-11 of the tanh value:
// a few 1e-3 in a logit of ordinary size, 0.024 at the cap of 50), the 32-bit path and the
// decode kernel use the exact form.  Every mbarrier wait is bounded in time.
//
// A second kernel further down runs the same walk on pairs of SMs for head sizes 128 and 256.
//
// The one-SM kernel has a second form (PAGED) for sequences that go on by many tokens: queries are the
// step's rows, at the positions the step gives them; a key tile is a page of the cache.  In the cache the
// 16-byte groups of row r of a [64][head_dim] tile are XOR-permuted by (r & 7), which within every 128-byte
// column block is exactly the 128-byte swizzle that the tensor core's operand descriptors expect: a page's
// tile is brought in by TMA boxes of [64 rows x 64 columns] WITHOUT swizzle and used as it lands.
//
// Compiled per head size: -DHOS_HEAD_DIM=N; the kernel exists for N in {64, 128, 256}.
#include <cuda.h>
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_utils.cuh"
#include "tcgen05_pair.cuh"

#ifndef HOS_HEAD_DIM
#define HOS_HEAD_DIM 64
#endif

namespace hos {

constexpr int THD = HOS_HEAD_DIM;
constexpr bool kHasTcPrefill = (THD == 64 || THD == 128 || THD == 256);

#if (HOS_HEAD_DIM == 64) || (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)

constexpr int TQ = 128, TK = 64;
constexpr int CBLK = THD / 64;                         // 64-element (128-byte) column blocks of a head
constexpr int kQBlockBytes = TQ * 128;                 // one column block of the Q tile
constexpr int kKVBlockBytes = TK * 128;                // one column block of a K or V tile
constexpr int kQBytesTc = CBLK * kQBlockBytes;
constexpr int kKVTileBytes = CBLK * kKVBlockBytes;
constexpr int kPBytes = TQ * 128;                      // 128 rows x 64 keys bf16
constexpr int kKVStages = 2;
constexpr int kXchgBytes = 2 * TQ * 4;                 // one float per (half, row)
constexpr int kTcSmem = kQBytesTc + kKVStages * 2 * kKVTileBytes + 2 * kPBytes + kXchgBytes + 160 + 976;
constexpr int kTcThreads = 320;                        // TMA warp, MMA warp, 8 softmax warps
constexpr int kTmemColsTc = (128 + THD) <= 256 ? 256 : 512;
constexpr int kColS = 0, kColO = 128;
constexpr long long kTcWaitCycles = 1ll << 31;
constexpr float kRescaleSlack = 8.0f;

__device__ int g_prefill_tc_error = 0;
__device__ int* g_prefill_tc_error_host = nullptr;     // a word in pinned host memory, if the host gave one

__device__ __forceinline__ void record_give_up() {
    atomicExch(&g_prefill_tc_error, 1);
    int* w = g_prefill_tc_error_host;
    if (w != nullptr) {
        atomicExch_system(w, kGiveUpAttnPrefill);
        __threadfence_system();
    }
}

__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > kTcWaitCycles) return false;
    return true;
}
__device__ __forceinline__ void tc_tma_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- tanh and exp2 shared between the MUFU unit and the FMA pipe ----------------------------------
// Per score the softmax needs a tanh (soft-cap) and an exp2, and the special-function unit takes 16 a clock
// per SM: with two softmax warps on a scheduler that unit, not the issue slots, sets the pace.  So a fixed
// share of a thread's scores (by index, no divergence) goes through polynomials on the FMA pipe instead:
//   tanh(x) = x + x^3 (a + x^2 (b + x^2 c)) for |x| <= 0.55, relative error 1.3e-6 (tanh.approx: 5e-4); a thread
//   whose polynomial scores are not all that small (a warp vote) takes the unit for all of them;
//   2^x = 2^n p(f), n = round(x), f = x - n in [-0.5, 0.5], p of degree 3 with relative error 7.5e-5 (the
//   result is rounded to bfloat16, 4e-3, for the product with V and summed as it stands), n added to the
//   exponent bits.
constexpr float kTanhPolyMax = 0.55f;
__device__ __forceinline__ float tanh_poly(float x) {
    const float x2 = x * x;
    float q = fmaf(-0.043099623f, x2, 0.13152355f);
    q = fmaf(q, x2, -0.33324513f);
    return fmaf(q * x2, x, x);
}
__device__ __forceinline__ float tanh_unit(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
    return t;
}
__device__ __forceinline__ float exp2_unit(float x) {
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(x));
    return p;
}
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -125.f);                                    // also what a masked score (-inf) becomes: 2^-125
    const float xr = x + 12582912.f;                         // 1.5 * 2^23: the low mantissa bits now hold round(x)
    const float f = x - (xr - 12582912.f);
    float p = fmaf(0.055171646f, f, 0.24261113f);
    p = fmaf(p, f, 0.69326097f);
    p = fmaf(p, f, 0.99992806f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(xr) << 23));
}
// Shares measured at head size 256, 8,192 tokens (us per launch; none: 258.9): tanh 3/8 alone 244.6, exp2 2/8 alone
// 251.8, 3/8 + 2/8 240.5, 4/8 + 2/8 240.1, 4/8 + 3/8 243.0, 5/8 + 3/8 253.3.
__device__ __forceinline__ bool tanh_by_poly(int i) { return (i & 7) < 4; }
__device__ __forceinline__ bool exp2_by_poly(int i) { return ((i >> 1) & 7) < 2; }
// t[i] = tanh(t[i] * pre) for a thread's N scores
template <int N>
__device__ __forceinline__ void tanh_scores(float (&t)[N], float pre) {
    float big = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        t[i] *= pre;
        if (tanh_by_poly(i)) big = fmaxf(big, fabsf(t[i]));
    }
    if (__any_sync(0xffffffffu, !(big <= kTanhPolyMax))) {          // a large (or not-a-number) score: the unit for all
#pragma unroll
        for (int i = 0; i < N; ++i) t[i] = tanh_unit(t[i]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) t[i] = tanh_by_poly(i) ? tanh_poly(t[i]) : tanh_unit(t[i]);
    }
}

// K-major tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major tile (the N dimension contiguous), 128-byte swizzle: a [K rows][64 N elements] block has rows
// of 128 bytes; 8-row K groups are 1024 bytes apart (stride offset), 64-element N blocks `block_bytes`
// apart (leading offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t block_bytes) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(block_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// bf16 x bf16 -> f32; b_mn: B operand is MN-major.
__host__ __device__ constexpr uint32_t tc_idesc(int m, int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

struct PrefillTcArgs {
    bf16* out;
    int out_stride;
    const int* cu_seqlens;
    int n_seqs, n_heads, n_kv_heads;
    int q_col0, k_col0, v_col0;     // first column of the q, k and v heads in a projection row
    float scale, cap;
    int window;
    // the paged form: sequence s has the rows cu_seqlens[s] - row_base .. of the query rows and of out, the first of
    // them at position token_pos[that row]; its keys and values are the pages of the table row seq_slot[s]
    int row_base;
    const int* token_pos;
    const int* seq_slot;
    const int* page_table;
    int table_stride, ring_pages;
};

// PAGED: map_kv covers the key pages and map_v the value pages, both as [pages x kv heads x 64 rows][head_dim]
// without swizzle; otherwise map_kv covers the projection rows (keys and values) and map_v is not used.
template <bool PAGED>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,      // boxes of [128 rows x 64 columns]
                       const __grid_constant__ CUtensorMap map_kv,     // boxes of [64 rows x 64 columns]
                       const __grid_constant__ CUtensorMap map_v,
                       PrefillTcArgs a) {
    // The kernel may start while the projection before it still runs: barriers, tensor memory and the look-ups of
    // the step's own arrays (written at the head of the step) are set up meanwhile; the producer waits for that
    // kernel's end before its first copy, and nothing else here touches global memory before data has arrived.
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* kv_s = q_s + kQBytesTc;                       // stage s: K tile then V tile
    unsigned char* p_s = kv_s + kKVStages * 2 * kKVTileBytes;
    float* xchg = reinterpret_cast<float*>(p_s + 2 * kPBytes);                 // [2 halves][128 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * kPBytes + kXchgBytes);
    uint64_t* q_full = bars;                 // 1
    uint64_t* k_full = bars + 1;             // [2] keys of a stage have landed
    uint64_t* k_empty = bars + 3;            // [2] S of that stage has been computed: its keys may be replaced
    uint64_t* s_full = bars + 5;             // [2]
    uint64_t* s_empty = bars + 7;            // [2]
    uint64_t* p_full = bars + 9;             // [2] one per P buffer
    uint64_t* pv_done = bars + 11;           // [2] one per P buffer
    uint64_t* v_full = bars + 13;            // [2] values of a stage have landed
    uint64_t* v_empty = bars + 15;           // [2] P.V of that stage is done: its values may be replaced
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 17);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which sequence and which block of 128 queries.  Long blocks first (late queries have most keys), and the
    // heads are the fast index of the grid: every head's longest walk starts in the first wave, and the heads
    // that share keys run side by side.
    int seq = 0, tile = blockIdx.y, row0 = 0, len = 0, nt = 0;
    for (; seq < a.n_seqs; ++seq) {
        row0 = a.cu_seqlens[seq] - (PAGED ? a.row_base : 0);
        len = a.cu_seqlens[seq + 1] - (PAGED ? a.row_base : 0) - row0;
        nt = (len + TQ - 1) / TQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (seq >= a.n_seqs) return;
    const int q0 = (nt - 1 - tile) * TQ;                    // first query row of the block within its sequence's rows
    const int p0 = q0 + (PAGED ? a.token_pos[row0] : 0);    // and its position
    const int head = blockIdx.x, kvh = head / (a.n_heads / a.n_kv_heads);
    const int last_q = p0 + min(len - 1 - q0, TQ - 1);
    const int first_key = a.window > 0 ? max(0, p0 + 1 - a.window) : 0;
    const int kt_lo = first_key / TK, kt_hi = last_q / TK;
    const int n_tiles = kt_hi - kt_lo + 1;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_kv)) : "memory");
        if (PAGED) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 8);
            mbar_init(&p_full[s], 8); mbar_init(&pv_done[s], 1);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_smem)),
                     "r"(kTmemColsTc) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            pdl_wait();       // the projection's rows and the step's keys and values are complete from here on
            mbar_expect_tx(q_full, kQBytesTc);
            for (int c = 0; c < CBLK; ++c)
                tc_tma_2d(q_s + c * kQBlockBytes, &map_q, a.q_col0 + head * THD + 64 * c, row0 + q0, q_full);
            // keys and values travel separately: a stage's keys are free again as soon as its S is
            // computed, long before its values are, so the next keys are fetched that much earlier
            PagedKV geo{nullptr, nullptr, a.page_table, a.table_stride, a.ring_pages, a.n_kv_heads, THD};
            const int* table = PAGED ? a.page_table + (size_t)a.seq_slot[seq] * a.table_stride : nullptr;
            int next_page = PAGED ? table[kv_table_entry(geo, kt_lo)] : 0;      // looked up one tile ahead of its use
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % kKVStages;
                unsigned char* kd = kv_s + (size_t)s * 2 * kKVTileBytes;
                unsigned char* vd = kd + kKVTileBytes;
                const int page = next_page;
                if (PAGED && j + 1 < n_tiles) next_page = table[kv_table_entry(geo, kt_lo + j + 1)];
                // the tile's first row in its tensor map, and the first column of its keys and of its values
                const int krow = PAGED ? (page * a.n_kv_heads + kvh) * kPageTokens : row0 + (kt_lo + j) * TK;
                const int kcol = PAGED ? 0 : a.k_col0 + kvh * THD, vcol = PAGED ? 0 : a.v_col0 + kvh * THD;
                if (j >= kKVStages && !tc_wait(&k_empty[s], ((j / kKVStages) - 1) & 1)) { ok = false; break; }
                mbar_expect_tx(&k_full[s], kKVTileBytes);
                for (int c = 0; c < CBLK; ++c)
                    tc_tma_2d(kd + c * kKVBlockBytes, &map_kv, kcol + 64 * c, krow, &k_full[s]);
                if (j >= kKVStages && !tc_wait(&v_empty[s], ((j / kKVStages) - 1) & 1)) { ok = false; break; }
                mbar_expect_tx(&v_full[s], kKVTileBytes);
                for (int c = 0; c < CBLK; ++c)
                    tc_tma_2d(vd + c * kKVBlockBytes, PAGED ? &map_v : &map_kv, vcol + 64 * c, krow, &v_full[s]);
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = tc_idesc(TQ, TK, 0);        // S = Q K^T: both K-major
            constexpr uint32_t idesc_o = tc_idesc(TQ, THD, 1);       // O = P V: V is MN-major
            bool ok = tc_wait(q_full, 0);
            tc_fence_after_sync();
            auto issue_s = [&](int j) -> bool {
                const int s = j % kKVStages, sb = j & 1;
                if (!tc_wait(&k_full[s], (j / kKVStages) & 1)) return false;
                if (j >= 2 && !tc_wait(&s_empty[sb], ((j >> 1) - 1) & 1)) return false;
                tc_fence_after_sync();
                const uint32_t k_addr = smem_u32(kv_s + (size_t)s * 2 * kKVTileBytes);
#pragma unroll
                for (int kk = 0; kk < THD / 16; ++kk) {
                    const uint64_t ad = desc_kmajor(smem_u32(q_s) + (kk / 4) * kQBlockBytes) + 2 * (kk % 4);
                    const uint64_t bd = desc_kmajor(k_addr + (kk / 4) * kKVBlockBytes) + 2 * (kk % 4);
                    tc_mma(tmem_base + kColS + sb * TK, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(&s_full[sb]);
                tc_commit(&k_empty[s]);       // the keys of this stage have been read
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }      // the next S runs under this tile's softmax
                const int pb = j & 1;
                if (!tc_wait(&p_full[pb], (j >> 1) & 1)) { ok = false; break; }
                const int s = j % kKVStages;
                if (!tc_wait(&v_full[s], (j / kKVStages) & 1)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t v_addr = smem_u32(kv_s + (size_t)s * 2 * kKVTileBytes + kKVTileBytes);
#pragma unroll
                for (int ks = 0; ks < TK / 16; ++ks) {
                    const uint64_t ad = desc_kmajor(smem_u32(p_s) + pb * kPBytes) + 2 * ks;
                    const uint64_t bd = desc_mnmajor(v_addr + ks * 16 * 128, kKVBlockBytes);
                    tc_mma(tmem_base + kColO, ad, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(&v_empty[s]);       // the values of this stage have been read
                tc_commit(&pv_done[pb]);      // this P buffer has been read, O holds tile j
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else {
        // ---------------- softmax, correction, epilogue: two threads per query row ----------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                        // which 32 of the tile's 64 keys
        const int r = quarter * 32 + lane;                       // row of the tile = TMEM lane
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int qpos = p0 + r;
        // The walk works on t = tanh(s * scale / cap) (or t = s without a cap): the logit is c * t with c = cap
        // (or scale), so the maximum is taken over t and a probability is exp2(t * c log2e - m * c log2e):
        // per score one multiply, tanh, maximum; one fused multiply-add, exp2, add.
        const bool capped = a.cap > 0.f;
        const float pre = capped ? a.scale / a.cap : 1.f;       // what the raw score is multiplied with before tanh
        const float c_logit = capped ? a.cap : a.scale;         // logit = c_logit * t
        const float c2 = c_logit * 1.4426950408889634f;
        const float slack_t = kRescaleSlack / c_logit;
        float m_ref = -INFINITY, l_run = 0.f;                    // m_ref in units of t; l_run: this thread's keys only
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j & 1, pb = j & 1;
            if (!tc_wait(&s_full[sb], (j >> 1) & 1)) { ok = false; break; }
            tc_fence_after_sync();
            float sc[32];
            {
                uint32_t v0[32];
                tc_ld32(t_lane + kColS + sb * TK + 32 * half, v0);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[i] = __uint_as_float(v0[i]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[sb]);            // this warp has its part of the S buffer
            const int kt0 = (kt_lo + j) * TK;                    // first key of the tile
            const int k0 = kt0 + 32 * half;
            float m_half = -INFINITY;
            if (capped) tanh_scores<32>(sc, pre);
            // a tile that every query of the block sees whole needs no mask (all but the last one or two of a walk,
            // and the first ones under a window)
            const bool whole = kt0 + TK - 1 <= p0 && (a.window <= 0 || kt0 > p0 + TQ - 1 - a.window);
            if (whole) {
#pragma unroll
                for (int i = 0; i < 32; ++i) m_half = fmaxf(m_half, sc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = k0 + i;
                    const bool vis = key <= qpos && (a.window <= 0 || key > qpos - a.window);
                    sc[i] = vis ? sc[i] : -INFINITY;
                    m_half = fmaxf(m_half, sc[i]);
                }
            }
            // the row's maximum over both halves
            xchg[half * TQ + r] = m_half;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float m_tile = fmaxf(m_half, xchg[(half ^ 1) * TQ + r]);
            asm volatile("bar.sync 1, 256;" ::: "memory");       // both have read before the next tile writes
            // raise the reference maximum only when it is exceeded by a margin (both threads of a row decide alike)
            float factor = 1.f;
            if (m_tile > m_ref + slack_t || (m_ref == -INFINITY && m_tile > -INFINITY)) {
                factor = m_ref == -INFINITY ? 0.f : __expf((m_ref - m_tile) * c_logit);
                m_ref = m_tile;
            }
            const float m_use2 = (m_ref == -INFINITY ? 0.f : m_ref) * c2;
            float psum = 0.f;
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float e0 = fmaf(sc[i], c2, -m_use2), e1 = fmaf(sc[i + 1], c2, -m_use2);
                const float p0 = exp2_by_poly(i) ? exp2_poly(e0) : exp2_unit(e0);
                const float p1 = exp2_by_poly(i + 1) ? exp2_poly(e1) : exp2_unit(e1);
                psum += p0 + p1;
                packed[i / 2] = pack_bf16(p0, p1);
            }
            l_run = l_run * factor + psum;
            // this P buffer is free once the product of two tiles ago has read it
            if (j >= 2 && !tc_wait(&pv_done[pb], ((j >> 1) - 1) & 1)) { ok = false; break; }
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // O is touched only between products: wait for the one of the tile before
                if (!tc_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = half * (THD / 2); c < (half + 1) * (THD / 2); c += 32) {
                    uint32_t o[32];
                    tc_ld32(t_lane + kColO + c, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tc_st32(t_lane + kColO + c, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // P row r, this thread's 32 keys: chunks 4*half .. 4*half+3 of 16 bytes, chunk c at position c ^ (r & 7)
            {
                unsigned char* prow = p_s + (size_t)pb * kPBytes + (size_t)r * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(prow + (((4 * half + c) ^ (r & 7)) << 4)) =
                        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes -> visible to the tensor core
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[pb]);
        }
        // ---- epilogue: O / l -> bfloat16 -> global; each thread half of its row ----
        if (ok && !tc_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1)) ok = false;
        if (ok) {
            tc_fence_after_sync();
            asm volatile("bar.sync 1, 256;" ::: "memory");      // every reader of xchg's maxima is done
            xchg[half * TQ + r] = l_run;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float l_row = l_run + xchg[(half ^ 1) * TQ + r];
            const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
            bf16* orow = a.out + (size_t)(row0 + q0 + r) * a.out_stride + (size_t)head * THD;
#pragma unroll 1
            for (int c = half * (THD / 2); c < (half + 1) * (THD / 2); c += 32) {
                uint32_t o[32];
                tc_ld32(t_lane + kColO + c, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (q0 + r < len) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        dst[q4] = make_uint4(
                            pack_bf16(__uint_as_float(o[8 * q4]) * inv, __uint_as_float(o[8 * q4 + 1]) * inv),
                            pack_bf16(__uint_as_float(o[8 * q4 + 2]) * inv, __uint_as_float(o[8 * q4 + 3]) * inv),
                            pack_bf16(__uint_as_float(o[8 * q4 + 4]) * inv, __uint_as_float(o[8 * q4 + 5]) * inv),
                            pack_bf16(__uint_as_float(o[8 * q4 + 6]) * inv, __uint_as_float(o[8 * q4 + 7]) * inv));
                }
            }
        }
        if (!ok && lane == 0) record_give_up();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsTc) : "memory");
}

// ---- the same walk on pairs of SMs (head sizes 128 and 256) ----------------------------------------
// With one CTA per block of queries every CTA streams all of its keys and values from L2, and at
// head size 256 that traffic (64 KB per 128 x 64 tile) is what bounds the kernel once the SMs are
// full.  Here the two query heads that share a kv head (an even number of heads per group) run as a
// pair of CTAs on the same block of 128 queries: one MMA of M = 256 (tcgen05 cta_group::2) covers
// both heads' queries, each CTA loads half of every key tile (64 of its 128 keys) and half of every
// value tile (half of the head's dimensions), so a key or value byte is fetched once for 256 query
// rows, and the tiles are 128 keys wide (S: 128 columns of tensor memory, twice, beside O).
// Each CTA's softmax warps work on their own head exactly as in the one-CTA kernel, a thread on 64
// keys of a tile.  Who signals whom (barriers at the same offsets in both CTAs):
//   q_full, k_full[s], v_full[s]   the leader's; its producer expects both CTAs' bytes
//   k_empty[s], v_empty[s], s_full[b], pv_done[b]   one per CTA, by the leader's multicast commit
//   s_empty[b], p_full[b]          the leader's; the 16 softmax warps of both CTAs arrive on it
#if (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)
constexpr int PK = 128;                                       // keys per tile
constexpr int kPairKBlockBytes = 64 * 128;                    // this CTA's 64 keys, one column block
constexpr int kPairKBytes = CBLK * kPairKBlockBytes;
constexpr int kPairVBlockBytes = PK * 128;                    // 128 keys, one column block of 64 dimensions
constexpr int kPairVBytes = (CBLK / 2) * kPairVBlockBytes;    // this CTA's half of the head's dimensions
constexpr int kPairStageBytes = kPairKBytes + kPairVBytes;
constexpr int kPairStages = 2;
constexpr int kPairPBlockBytes = TQ * 128;                    // 128 rows x 64 keys
constexpr int kPairPBytes = 2 * kPairPBlockBytes;
constexpr int kPairPBufs = THD == 256 ? 1 : 2;                // what shared memory has room for
constexpr int kPairSmem = kQBytesTc + kPairStages * kPairStageBytes + kPairPBufs * kPairPBytes + kXchgBytes + 160 + 976;
constexpr int kPairColS = 0, kPairColO = 2 * PK;
constexpr int kPairTmemCols = 512;
static_assert(kPairSmem <= 232448, "the pair kernel's shared memory");
static_assert(kPairColO + THD <= kPairTmemCols, "the pair kernel's tensor memory");

__device__ __forceinline__ bool tc_wait_cluster(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait_cluster(bar, parity))
        if (clock64() - t0 > kTcWaitCycles) return false;
    return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTcThreads, 1)
attn_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q,      // boxes of [128 rows x 64 columns]
                         const __grid_constant__ CUtensorMap map_k,      // boxes of [64 rows x 64 columns]
                         PrefillTcArgs a) {
    pdl_launch_dependents();      // as in the one-CTA kernel: set-up first, the producers wait before their first copy
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* kv_s = q_s + kQBytesTc;                       // stage s: this CTA's keys, then its part of the values
    unsigned char* p_s = kv_s + kPairStages * kPairStageBytes;
    float* xchg = reinterpret_cast<float*>(p_s + kPairPBufs * kPairPBytes);    // [2 halves][128 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + kPairPBufs * kPairPBytes + kXchgBytes);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 3;
    uint64_t* s_full = bars + 5;
    uint64_t* s_empty = bars + 7;
    uint64_t* p_full = bars + 9;
    uint64_t* pv_done = bars + 11;
    uint64_t* v_full = bars + 13;
    uint64_t* v_empty = bars + 15;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 17);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;

    // which sequence and which block of 128 queries: the same for both CTAs of a pair (they differ in the head)
    int seq = 0, tile = blockIdx.y, row0 = 0, len = 0, nt = 0;
    for (; seq < a.n_seqs; ++seq) {
        row0 = a.cu_seqlens[seq];
        len = a.cu_seqlens[seq + 1] - row0;
        nt = (len + TQ - 1) / TQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (seq >= a.n_seqs) return;                                 // both CTAs of the pair alike
    const int q0 = (nt - 1 - tile) * TQ;
    const int head = blockIdx.x, kvh = head / (a.n_heads / a.n_kv_heads);
    const int last_q = min(len - 1, q0 + TQ - 1);
    const int first_key = a.window > 0 ? max(0, q0 + 1 - a.window) : 0;
    const int kt_lo = first_key / PK, kt_hi = last_q / PK;
    const int n_tiles = kt_hi - kt_lo + 1;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 16);
            mbar_init(&p_full[s], 16); mbar_init(&pv_done[s], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();
    cluster_sync_all();                                          // both CTAs' barriers exist before anything arrives on them
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_smem, kPairTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs, each its own halves) ----------------
        if (lane == 0) {
            bool ok = true;
            pdl_wait();       // the projection's rows are complete from here on
            if (leader) mbar_expect_tx(q_full, 2 * kQBytesTc);
            for (int c = 0; c < CBLK; ++c)
                tma_load_2d_pair(q_s + c * kQBlockBytes, &map_q, a.q_col0 + head * THD + 64 * c, row0 + q0, q_full);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % kPairStages;
                unsigned char* kd = kv_s + (size_t)s * kPairStageBytes;
                unsigned char* vd = kd + kPairKBytes;
                const int krow = row0 + (kt_lo + j) * PK;
                if (j >= kPairStages && !tc_wait(&k_empty[s], ((j / kPairStages) - 1) & 1)) { ok = false; break; }
                if (leader) mbar_expect_tx(&k_full[s], 2 * kPairKBytes);
                for (int c = 0; c < CBLK; ++c)          // keys 64 rank .. 64 rank + 63 of the tile, all dimensions
                    tma_load_2d_pair(kd + c * kPairKBlockBytes, &map_k, a.k_col0 + kvh * THD + 64 * c, krow + 64 * (int)rank,
                                     &k_full[s]);
                if (j >= kPairStages && !tc_wait(&v_empty[s], ((j / kPairStages) - 1) & 1)) { ok = false; break; }
                if (leader) mbar_expect_tx(&v_full[s], 2 * kPairVBytes);
                for (int c = 0; c < CBLK / 2; ++c)      // all 128 keys, this CTA's half of the dimensions
                    tma_load_2d_pair(vd + c * kPairVBlockBytes, &map_q, a.v_col0 + kvh * THD + (THD / 2) * (int)rank + 64 * c, krow,
                                     &v_full[s]);
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread of the leader, for both CTAs ----------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc_s = tc_idesc(2 * TQ, PK, 0);        // S = Q K^T: both K-major
            constexpr uint32_t idesc_o = tc_idesc(2 * TQ, THD, 1);       // O = P V: V is MN-major
            bool ok = tc_wait(q_full, 0);
            tc_fence_after_sync();
            auto issue_s = [&](int j) -> bool {
                const int s = j % kPairStages, sb = j & 1;
                if (!tc_wait(&k_full[s], (j / kPairStages) & 1)) return false;
                if (j >= 2 && !tc_wait_cluster(&s_empty[sb], ((j >> 1) - 1) & 1)) return false;
                tc_fence_after_sync();
                const uint32_t k_addr = smem_u32(kv_s + (size_t)s * kPairStageBytes);
#pragma unroll
                for (int kk = 0; kk < THD / 16; ++kk) {
                    const uint64_t ad = desc_kmajor(smem_u32(q_s) + (kk / 4) * kQBlockBytes) + 2 * (kk % 4);
                    const uint64_t bd = desc_kmajor(k_addr + (kk / 4) * kPairKBlockBytes) + 2 * (kk % 4);
                    umma_bf16_pair(tmem_base + kPairColS + sb * PK, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit_pair(&s_full[sb]);
                umma_commit_pair(&k_empty[s]);      // the keys of this stage have been read
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }      // the next S runs under this tile's softmax
                const int pb = j % kPairPBufs;
                if (!tc_wait_cluster(&p_full[pb], (j / kPairPBufs) & 1)) { ok = false; break; }
                const int s = j % kPairStages;
                if (!tc_wait(&v_full[s], (j / kPairStages) & 1)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t v_addr = smem_u32(kv_s + (size_t)s * kPairStageBytes + kPairKBytes);
#pragma unroll
                for (int ks = 0; ks < PK / 16; ++ks) {
                    const uint64_t ad = desc_kmajor(smem_u32(p_s) + pb * kPairPBytes + (ks / 4) * kPairPBlockBytes) + 2 * (ks % 4);
                    const uint64_t bd = desc_mnmajor(v_addr + ks * 16 * 128, kPairVBlockBytes);
                    umma_bf16_pair(tmem_base + kPairColO, ad, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit_pair(&v_empty[s]);      // the values of this stage have been read
                umma_commit_pair(&pv_done[pb]);     // this P buffer has been read, O holds tile j
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else {
        // ---------------- softmax, correction, epilogue: two threads per query row, 64 keys each ----------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                        // which 64 of the tile's 128 keys
        const int r = quarter * 32 + lane;                       // row of the tile = TMEM lane
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int qpos = q0 + r;
        const bool capped = a.cap > 0.f;
        const float pre = capped ? a.scale / a.cap : 1.f;
        const float c_logit = capped ? a.cap : a.scale;          // logit = c_logit * t
        const float c2 = c_logit * 1.4426950408889634f;
        const float slack_t = kRescaleSlack / c_logit;
        float m_ref = -INFINITY, l_run = 0.f;                    // m_ref in units of t; l_run: this thread's keys only
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j & 1, pb = j % kPairPBufs;
            if (!tc_wait(&s_full[sb], (j >> 1) & 1)) { ok = false; break; }
            tc_fence_after_sync();
            float sc[64];
            {
                uint32_t v0[32], v1[32];
                tc_ld32(t_lane + kPairColS + sb * PK + 64 * half, v0);
                tc_ld32(t_lane + kPairColS + sb * PK + 64 * half + 32, v1);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) { sc[i] = __uint_as_float(v0[i]); sc[32 + i] = __uint_as_float(v1[i]); }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&s_empty[sb]);     // this warp has its part of the S buffer
            const int kt0 = (kt_lo + j) * PK;                    // first key of the tile
            const int k0 = kt0 + 64 * half;
            if (capped) tanh_scores<64>(sc, pre);
            float m_half = -INFINITY;
            const bool whole = kt0 + PK - 1 <= q0 && (a.window <= 0 || kt0 > q0 + TQ - 1 - a.window);
            if (whole) {
#pragma unroll
                for (int i = 0; i < 64; ++i) m_half = fmaxf(m_half, sc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = k0 + i;
                    const bool vis = key <= qpos && (a.window <= 0 || key > qpos - a.window);
                    sc[i] = vis ? sc[i] : -INFINITY;
                    m_half = fmaxf(m_half, sc[i]);
                }
            }
            xchg[half * TQ + r] = m_half;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float m_tile = fmaxf(m_half, xchg[(half ^ 1) * TQ + r]);
            asm volatile("bar.sync 1, 256;" ::: "memory");       // both have read before the next tile writes
            float factor = 1.f;
            if (m_tile > m_ref + slack_t || (m_ref == -INFINITY && m_tile > -INFINITY)) {
                factor = m_ref == -INFINITY ? 0.f : __expf((m_ref - m_tile) * c_logit);
                m_ref = m_tile;
            }
            const float m_use2 = (m_ref == -INFINITY ? 0.f : m_ref) * c2;
            float psum = 0.f;
            uint32_t packed[32];
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const float e0 = fmaf(sc[i], c2, -m_use2), e1 = fmaf(sc[i + 1], c2, -m_use2);
                const float p0 = exp2_by_poly(i) ? exp2_poly(e0) : exp2_unit(e0);
                const float p1 = exp2_by_poly(i + 1) ? exp2_poly(e1) : exp2_unit(e1);
                psum += p0 + p1;
                packed[i / 2] = pack_bf16(p0, p1);
            }
            l_run = l_run * factor + psum;
            // this P buffer is free once the product that read it last is done
            if (j >= kPairPBufs && !tc_wait(&pv_done[pb], ((j / kPairPBufs) - 1) & 1)) { ok = false; break; }
            if (j > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
                // O is touched only between products: wait for the one of the tile before
                if (!tc_wait(&pv_done[(j - 1) % kPairPBufs], ((j - 1) / kPairPBufs) & 1)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll 1
                for (int c = half * (THD / 2); c < (half + 1) * (THD / 2); c += 32) {
                    uint32_t o[32];
                    tc_ld32(t_lane + kPairColO + c, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                    tc_st32(t_lane + kPairColO + c, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // P row r, this thread's 64 keys = column block `half`: chunk c of 16 bytes at position c ^ (r & 7)
            {
                unsigned char* prow = p_s + (size_t)pb * kPairPBytes + (size_t)half * kPairPBlockBytes + (size_t)r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) =
                        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            // The proxy fence makes this thread's P visible to the tensor core of its own SM, which is the one that
            // reads it (the A rows of an MMA on a pair come from each CTA's own shared memory); the arrival on the
            // leader's barrier is the plain one: with release semantics over the cluster this step took 1,400 cycles
            // instead of 490 per tile.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&p_full[pb]);
        }
        // ---- epilogue: O / l -> bfloat16 -> global; each thread half of its row ----
        if (ok && !tc_wait(&pv_done[(n_tiles - 1) % kPairPBufs], ((n_tiles - 1) / kPairPBufs) & 1)) ok = false;
        if (ok) {
            tc_fence_after_sync();
            asm volatile("bar.sync 1, 256;" ::: "memory");      // every reader of xchg's maxima is done
            xchg[half * TQ + r] = l_run;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float l_row = l_run + xchg[(half ^ 1) * TQ + r];
            const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
            bf16* orow = a.out + (size_t)(row0 + qpos) * a.out_stride + (size_t)head * THD;
#pragma unroll 1
            for (int c = half * (THD / 2); c < (half + 1) * (THD / 2); c += 32) {
                uint32_t o[32];
                tc_ld32(t_lane + kPairColO + c, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (qpos < len) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        dst[q4] = make_uint4(
                            pack_bf16(__uint_as_float(o[8 * q4]) * inv, __uint_as_float(o[8 * q4 + 1]) * inv),
                            pack_bf16(__uint_as_float(o[8 * q4 + 2]) * inv, __uint_as_float(o[8 * q4 + 3]) * inv),
                            pack_bf16(__uint_as_float(o[8 * q4 + 4]) * inv, __uint_as_float(o[8 * q4 + 5]) * inv),
                            pack_bf16(__uint_as_float(o[8 * q4 + 6]) * inv, __uint_as_float(o[8 * q4 + 7]) * inv));
                }
            }
        }
        if (!ok && lane == 0) record_give_up();
    }
    // ---- teardown: nobody of either CTA touches tensor memory or the other's barriers any more ----
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, kPairTmemCols);
}
#endif   // head sizes with the pair kernel

typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TcEncodeFn tc_encode_fn() {
    static TcEncodeFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TcEncodeFn>(sym);
    }
    return fn;
}
// swizzle: the 128-byte swizzle for rows as the projection wrote them; none for the cache's tiles, which lie
// permuted in memory the way the swizzle would place them
static int tc_make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, int ld, int box_rows,
                       bool swizzle = true) {
    TcEncodeFn fn = tc_encode_fn();
    if (!fn) HOS_REFUSE("attn_prefill_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HOS_REFUSE("attn_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}
#endif   // head sizes with the kernel

}  // namespace hos

using namespace hos;

// Whether prompts of models whose query heads share keys two by two run on pairs of SMs (head sizes
// 128 and 256).  Default on; HOS_ATTN_PAIR=0 in the environment or hos_attn_prefill_pair(0) switch it off.
static int& pair_state() {
    static int on = !(getenv("HOS_ATTN_PAIR") && getenv("HOS_ATTN_PAIR")[0] == '0');
    return on;
}
extern "C" int hos_attn_prefill_pair(int on) {
    pair_state() = on ? 1 : 0;
    return 0;
}

// 1 if this library has the tensor-core prompt kernel (head sizes 64, 128, 256).
extern "C" int hos_attn_prefill_tc_available() { return kHasTcPrefill ? 1 : 0; }

// The host's word for waits that ran out; null takes it away.
extern "C" int hos_attn_prefill_tc_set_error_word(int* word) {
#if (HOS_HEAD_DIM == 64) || (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)
    if (cudaMemcpyToSymbol(g_prefill_tc_error_host, &word, sizeof(word)) != cudaSuccess)
        HOS_REFUSE("attn_prefill_tc: cannot set the error word: %s", cudaGetErrorString(cudaGetLastError()));
#endif
    return 0;
}

// 1 if an earlier launch gave up a bounded wait (and clears the flag).  Synchronises.
extern "C" int hos_attn_prefill_tc_error() {
#if (HOS_HEAD_DIM == 64) || (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_prefill_tc_error, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_prefill_tc_error, &zero, sizeof(int));
    return v;
#else
    return 0;
#endif
}

// rows: the fused projection output [n_rows, row_stride] (q heads, then k heads, then v heads);
// sequences occupy rows cu_seqlens[s] .. cu_seqlens[s+1]-1, each from position 0; n_q_tiles is the
// sum over sequences of ceil(len / 128).
extern "C" int hos_attn_prefill_tc(const void* rows, long long n_rows, int row_stride, void* out, int out_stride,
                                   const int* cu_seqlens, int n_seqs, int n_q_tiles, int n_heads, int n_kv_heads,
                                   int head_dim, float scale, float cap, int window, cudaStream_t stream) {
#if (HOS_HEAD_DIM == 64) || (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)
    if (n_q_tiles <= 0 || n_seqs <= 0) return 0;
    if (head_dim != THD) HOS_REFUSE("attn_prefill_tc: built for head_dim %d, asked for %d", THD, head_dim);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_prefill_tc: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (n_q_tiles > 65535) HOS_REFUSE("attn_prefill_tc: %d blocks of queries are more than one launch takes", n_q_tiles);
    if (row_stride != (n_heads + 2 * n_kv_heads) * THD)
        HOS_REFUSE("attn_prefill_tc: a row of %d elements is not q, k and v heads of %d", row_stride, THD);
    if ((row_stride % 8) || ((uintptr_t)rows % 16) || (out_stride % 8) || ((uintptr_t)out % 16))
        HOS_REFUSE("attn_prefill_tc: rows must be 16-byte aligned");
    CUtensorMap mq, mkv;
    int rc;
    if ((rc = tc_make_map(&mq, rows, n_rows, row_stride, row_stride, TQ))) return rc;
    if ((rc = tc_make_map(&mkv, rows, n_rows, row_stride, row_stride, TK))) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess)
            HOS_REFUSE("attn_prefill_tc: cannot get %d bytes of shared memory", kTcSmem);
        attr_set = true;
    }
    PrefillTcArgs a = {};
    a.out = (bf16*)out; a.out_stride = out_stride; a.cu_seqlens = cu_seqlens; a.n_seqs = n_seqs;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads;
    a.q_col0 = 0; a.k_col0 = n_heads * THD; a.v_col0 = (n_heads + n_kv_heads) * THD;
    a.scale = scale; a.cap = cap; a.window = window;
    dim3 grid(n_heads, n_q_tiles);
#if (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)
    // pairs of SMs when two query heads share their keys (and nothing switched it off)
    if (pair_state() != 0 && (n_heads / n_kv_heads) % 2 == 0) {
        static bool pair_attr_set = false;
        if (!pair_attr_set) {
            if (cudaFuncSetAttribute(attn_prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) != cudaSuccess)
                HOS_REFUSE("attn_prefill_tc: cannot get %d bytes of shared memory", kPairSmem);
            pair_attr_set = true;
        }
        launch_pdl(attn_prefill_pair_kernel, dim3(grid), dim3(kTcThreads), kPairSmem, stream, mq, mkv, a);
        return check_launch("attn_prefill_tc (pairs of SMs)");
    }
#endif
    launch_pdl(attn_prefill_tc_kernel<false>, dim3(grid), dim3(kTcThreads), kTcSmem, stream, mq, mkv, mkv, a);
    return check_launch("attn_prefill_tc");
#else
    HOS_REFUSE("attn_prefill_tc: no tensor-core prompt kernel for head_dim %d (64, 128 and 256 have one)", HOS_HEAD_DIM);
#endif
}

// Sequences that go on by many tokens, over the paged cache (which holds the step's keys already), on the tensor
// cores.  q: the step's projection rows of these sequences [n_rows, row_stride] (the q heads stand first in a row);
// sequence s has the rows cu_seqlens[s] - row_base .. of q and out, at the consecutive positions token_pos[row], and
// the page-table row seq_slot[s]; n_q_tiles is at least the sum over sequences of ceil(rows / 128).  The pages are
// [n_pages][n_kv_heads][64][head_dim] arrays in the cache's permuted layout.
extern "C" int hos_attn_chunk_tc(const void* q, long long n_rows, int row_stride, void* out, int out_stride,
                                 const int* cu_seqlens, int row_base, const int* token_pos, const int* seq_slot,
                                 int n_seqs, int n_q_tiles, void* k_pages, void* v_pages, long long n_pages,
                                 const int* page_table, int table_stride, int ring_pages, int n_heads, int n_kv_heads,
                                 int head_dim, float scale, float cap, int window, cudaStream_t stream) {
#if (HOS_HEAD_DIM == 64) || (HOS_HEAD_DIM == 128) || (HOS_HEAD_DIM == 256)
    if (n_q_tiles <= 0 || n_seqs <= 0) return 0;
    if (head_dim != THD) HOS_REFUSE("attn_chunk_tc: built for head_dim %d, asked for %d", THD, head_dim);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        HOS_REFUSE("attn_chunk_tc: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (n_q_tiles > 65535) HOS_REFUSE("attn_chunk_tc: %d blocks of queries are more than one launch takes", n_q_tiles);
    if (row_stride < n_heads * THD || (row_stride % 8) || ((uintptr_t)q % 16) || (out_stride % 8) || ((uintptr_t)out % 16))
        HOS_REFUSE("attn_chunk_tc: rows must hold the q heads and be 16-byte aligned");
    if (((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || n_pages <= 0)
        HOS_REFUSE("attn_chunk_tc: the pages must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = tc_make_map(&mq, q, n_rows, row_stride, row_stride, TQ))) return rc;
    const long long page_rows = n_pages * n_kv_heads * kPageTokens;
    if ((rc = tc_make_map(&mk, k_pages, page_rows, THD, THD, TK, false))) return rc;
    if ((rc = tc_make_map(&mv, v_pages, page_rows, THD, THD, TK, false))) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(attn_prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem) != cudaSuccess)
            HOS_REFUSE("attn_chunk_tc: cannot get %d bytes of shared memory", kTcSmem);
        attr_set = true;
    }
    PrefillTcArgs a = {};
    a.out = (bf16*)out; a.out_stride = out_stride; a.cu_seqlens = cu_seqlens; a.n_seqs = n_seqs;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads;
    a.q_col0 = 0; a.k_col0 = 0; a.v_col0 = 0;
    a.scale = scale; a.cap = cap; a.window = window;
    a.row_base = row_base; a.token_pos = token_pos; a.seq_slot = seq_slot;
    a.page_table = page_table; a.table_stride = table_stride; a.ring_pages = ring_pages;
    launch_pdl(attn_prefill_tc_kernel<true>, dim3(n_heads, n_q_tiles), dim3(kTcThreads), kTcSmem, stream, mq, mk, mv, a);
    return check_launch("attn_chunk_tc");
#else
    HOS_REFUSE("attn_chunk_tc: no tensor-core kernel for head_dim %d (64, 128 and 256 have one)", HOS_HEAD_DIM);
#endif
}
