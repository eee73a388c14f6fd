// bfloat16 matrix product on the 5th-generation tensor cores: out[M, N] = A[M, K] . W[N, K]^T.
//
// Both operands are K-major (rows of K contiguous elements), which is how activations and
// checkpoint weights lie in memory.  TMA (cp.async.bulk.tensor, 128-byte swizzle) brings
// [rows x 64] tiles of both into shared memory through a ring of stages; one thread issues
// tcgen05.mma (M = 128, N = the other tile's rows, K = 16 per instruction) with the 32-bit
// accumulator in tensor memory; four warps read the accumulator back (tcgen05.ld), apply the
// epilogue and store.  The kernel is persistent: each CTA walks over output tiles, with two
// accumulators in tensor memory so that the epilogue of one tile overlaps the products of
// the next.  Warp roles: 0 TMA producer, 1 MMA issuer (and tensor-memory allocation), 2-5
// epilogue.
//
// Two orientations share the code.  "Normal": the 128-row MMA operand is a tile of A
// (tokens), the N operand 256 rows of W; thread t of the epilogue holds one token's row of
// the output tile.  "Swapped" (few tokens, e.g. decoding): the 128-row operand is a tile of W
// and the N operand is all of A's rows (16, 32 or 64); the accumulator holds the output
// transposed and the epilogue writes it back in place, coalesced over output features.  In
// the swapped orientation K may be split over several CTAs, each writing 32-bit partial sums
// that a small kernel adds in a fixed order.
//
// Epilogues: none; soft-cap c*tanh(x/c) with 32-bit output (logits); gated act(gate)*up,
// where W holds the gate rows followed by the up rows and a tile loads matching rows of both.
//
// Every wait on an mbarrier is bounded in time: a wait that runs out sets an error flag,
// the roles leave their loops, tensor memory is freed and the kernel returns.
#include <cuda.h>
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_utils.cuh"
#include "tcgen05_pair.cuh"

namespace hos {

constexpr int GM = 128;            // rows of the M operand per tile (UMMA M)
constexpr int GK = 64;             // K elements per stage: 128 bytes, one swizzle atom
constexpr int kGemmThreads = 192;
constexpr int kPairThreads = 320;         // the kernel on pairs of SMs: TMA warp, MMA warp, 8 epilogue warps
constexpr long long kWaitCycles = 1ll << 31;     // about a second

enum { kGEpiNone = 0, kGEpiSoftcap = 1, kGEpiGated = 2, kGEpiRope = 3 };

__device__ int g_gemm_error = 0;
__device__ int* g_gemm_error_host = nullptr;     // a word in pinned host memory, if the host gave one

// A wait ran out: the device flag for hos_gemm_tc_error(), and the host's word, which it can look at
// after any synchronisation without asking the device.
__device__ __forceinline__ void record_give_up() {
    atomicExch(&g_gemm_error, 1);
    int* w = g_gemm_error_host;
    if (w != nullptr) {
        atomicExch_system(w, kGiveUpGemmTc);
        __threadfence_system();
    }
}

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity, long long limit = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > limit) return false;
    return true;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base + i)'s columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (the tile base is 1024-byte aligned).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                               // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                               // layout: 128-byte swizzle
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// What the rotary epilogue of the q/k/v projection needs (kGEpiRope): the output's columns are q heads, then k
// heads, then v heads of head_dim each; q and k heads are rotated (rotate-half over the whole head: the pair
// (i, i + head_dim/2) by position * inv_freq[i]), and keys and values go to the tokens' places in the paged cache.
struct RopeEpi {
    const int* token_pos;
    const int* token_seq;
    const int* seq_slot;
    const int* seq_len_after;
    const float2* angles;      // [M][head_dim / 2] (cos, sin)
    PagedKV cache;
    int n_heads, n_kv_heads, write_cache;
};

struct GemmParams {
    void* out;            // [M, N] row-major (bf16 or f32); with K splits: f32 partials [splits][M][N]
    int M, N, K;          // the product's logical sizes: rows of A, rows of W (per half if gated), K
    int ldo;
    int k_splits;
    int gate_rows;        // gated: row of W where the up rows begin
    float cap;
    int act;
    RopeEpi rope;         // kGEpiRope only
};

template <int BN, bool SWAP>
struct GemmCfg {
    static constexpr int kABytes = GM * GK * 2;
    static constexpr int kBBytes = BN * GK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagesRaw = (196 * 1024) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static constexpr int kExchangeBytes = SWAP ? 64 * BN * 4 : 0;          // gated + swapped: up rows cross warps
    static constexpr int kSmem = kStages * kStageBytes + kExchangeBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;            // two accumulators; a power of two >= 32
};

template <int BN, int EPI, bool SWAP, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_m,     // the 128-row operand: A (normal) or W (swapped)
               const __grid_constant__ CUtensorMap map_n,     // the BN-row operand: W (normal) or A (swapped)
               GemmParams p) {
    using Cfg = GemmCfg<BN, SWAP>;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;
    float* exchange = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes + Cfg::kExchangeBytes);
    uint64_t* full = bars;                          // [kStages] TMA -> MMA
    uint64_t* empty = bars + Cfg::kStages;          // [kStages] MMA -> TMA
    uint64_t* acc_full = empty + Cfg::kStages;      // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;             // [2] epilogue -> MMA
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // rows of the two MMA operands in the product's terms
    const int rows_m = SWAP ? p.N : p.M;            // what the 128-row operand spans
    const int rows_n = SWAP ? p.M : p.N;
    const int m_tiles = (rows_m + (EPI == kGEpiGated && SWAP ? 64 : GM) - 1) / (EPI == kGEpiGated && SWAP ? 64 : GM);
    const int n_span = (EPI == kGEpiGated && !SWAP) ? BN / 2 : BN;        // output columns (normal) per tile
    const int n_tiles = (rows_n + n_span - 1) / n_span;
    const int k_blocks = (p.K + GK - 1) / GK;
    const int kb_per_split = (k_blocks + p.k_splits - 1) / p.k_splits;
    const int total_tiles = m_tiles * n_tiles * p.k_splits;

    if (threadIdx.x == 0) {
        prefetch_tmap(&map_m);
        prefetch_tmap(&map_n);
        for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_smem, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;
    pdl_enter();      // barriers and tensor memory were set up beside the tail of the kernel before; its results are read from here on

    auto tile_coords = [&](int tile, int& mt, int& nt, int& ks) {
        ks = tile % p.k_splits;
        const int t = tile / p.k_splits;
        mt = t % m_tiles;
        nt = t / m_tiles;
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int mt, nt, ks;
                tile_coords(tile, mt, nt, ks);
                const int kb0 = ks * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    if (it >= Cfg::kStages && !mbar_wait_timed(&empty[s], ((it / Cfg::kStages) - 1) & 1)) { ok = false; break; }
                    unsigned char* a_dst = stages + (size_t)s * Cfg::kStageBytes;
                    unsigned char* b_dst = a_dst + Cfg::kABytes;
                    mbar_expect_tx(&full[s], Cfg::kStageBytes);
                    if (EPI == kGEpiGated && SWAP) {        // 64 gate rows, then the 64 matching up rows
                        tma_load_2d(a_dst, &map_m, kb * GK, mt * 64, &full[s]);
                        tma_load_2d(a_dst + Cfg::kABytes / 2, &map_m, kb * GK, p.gate_rows + mt * 64, &full[s]);
                    } else {
                        tma_load_2d(a_dst, &map_m, kb * GK, mt * GM, &full[s]);
                    }
                    if (EPI == kGEpiGated && !SWAP) {       // BN/2 gate rows, then the matching up rows
                        tma_load_2d(b_dst, &map_n, kb * GK, nt * (BN / 2), &full[s]);
                        tma_load_2d(b_dst + Cfg::kBBytes / 2, &map_n, kb * GK, p.gate_rows + nt * (BN / 2), &full[s]);
                    } else {
                        tma_load_2d(b_dst, &map_n, kb * GK, nt * BN, &full[s]);
                    }
                }
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(GM, BN);
            int it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
                int mt, nt, ks;
                tile_coords(tile, mt, nt, ks);
                const int kb0 = ks * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
                const int acc = local_tile & 1;
                if (local_tile >= 2 && !mbar_wait_timed(&acc_empty[acc], ((local_tile >> 1) - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    if (!mbar_wait_timed(&full[s], (it / Cfg::kStages) & 1)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stages + (size_t)s * Cfg::kStageBytes);
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < GK / 16; ++k)     // 32 bytes further along K: +2 in 16-byte units
                        umma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);               // the stage is free once these products have read it
                }
                if (ok) umma_commit(&acc_full[acc]);      // the accumulator is complete
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warps 2..5, each owns the TMEM lanes 32*(warp%4).. ----------------
        const int quarter = warp & 3;
        int local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
            int mt, nt, ks;
            tile_coords(tile, mt, nt, ks);
            const int acc = local_tile & 1;
            if (!mbar_wait_timed(&acc_full[acc], (local_tile >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            const int r = quarter * 32 + lane;            // this thread's row of the accumulator
            if (!SWAP) {
                // row r = token mt*128 + r; columns = output features
                const int m = mt * GM + r;
                OutT* orow = reinterpret_cast<OutT*>(p.out) + (size_t)m * p.ldo;
                constexpr int COLS = (EPI == kGEpiGated) ? BN / 2 : BN;
#pragma unroll 1
                for (int c0 = 0; c0 < COLS; c0 += 32) {
                    uint32_t v[32], u[32];
                    tmem_ld_32x32(t_lane + c0, v);
                    if (EPI == kGEpiGated) tmem_ld_32x32(t_lane + BN / 2 + c0, u);
                    tmem_ld_wait();
                    const int n0 = nt * COLS + c0;
                    if (m < p.M) {
                        float f[32];
                        if (EPI == kGEpiGated) {
                            if (p.act == 0) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) f[j] = gelu_tanh_fast(__uint_as_float(v[j])) * __uint_as_float(u[j]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j) f[j] = silu_fast(__uint_as_float(v[j])) * __uint_as_float(u[j]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const float x = __uint_as_float(v[j]);
                                f[j] = EPI == kGEpiSoftcap ? softcap_precise(x, p.cap) : x;
                            }
                        }
                        if (n0 + 32 <= p.N && (p.ldo % 8) == 0) {
                            if (sizeof(OutT) == 2) {
                                uint4* dst = reinterpret_cast<uint4*>(orow + n0);
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    dst[q] = make_uint4(pack_bf16(f[8 * q], f[8 * q + 1]), pack_bf16(f[8 * q + 2], f[8 * q + 3]),
                                                        pack_bf16(f[8 * q + 4], f[8 * q + 5]), pack_bf16(f[8 * q + 6], f[8 * q + 7]));
                            } else {
                                float4* dst = reinterpret_cast<float4*>(orow + n0);
#pragma unroll
                                for (int q = 0; q < 8; ++q) dst[q] = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (n0 + j < p.N) orow[n0 + j] = from_float<OutT>(f[j]);
                        }
                    }
                }
            } else {
                // row r = output feature; columns = tokens.  out[token][feature]: a warp's 32
                // lanes write 32 consecutive features of one token.
                const bool gated = EPI == kGEpiGated;
                const int feat = gated ? mt * 64 + (r & 63) : mt * GM + r;
                const int feat_count = p.N;
                OutT* obase = reinterpret_cast<OutT*>(p.out) + (p.k_splits > 1 ? (size_t)ks * p.M * p.ldo : 0);
                constexpr int CH = BN < 32 ? BN : 32;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += CH) {
                    float f[CH];
                    if (CH == 32) {
                        uint32_t v[32];
                        tmem_ld_32x32(t_lane + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                    } else {
                        uint32_t v[16];
                        tmem_ld_32x16(t_lane + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < CH; ++j) f[j] = __uint_as_float(v[j]);
                    }
                    if (gated) {
                        // lanes 64..127 hold the up rows of the features whose gate rows lanes 0..63 hold
                        if (r >= 64) {
#pragma unroll
                            for (int j = 0; j < CH; ++j) exchange[(r - 64) * BN + c0 + j] = f[j];
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (r < 64) {
                            if (p.act == 0) {
#pragma unroll
                                for (int j = 0; j < CH; ++j) f[j] = gelu_tanh_fast(f[j]) * exchange[r * BN + c0 + j];
                            } else {
#pragma unroll
                                for (int j = 0; j < CH; ++j) f[j] = silu_fast(f[j]) * exchange[r * BN + c0 + j];
                            }
                        }
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (r >= 64) continue;
                    }
                    if (feat < feat_count) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            const int tok = nt * BN + c0 + j;
                            if (tok < p.M) {
                                float x = f[j];
                                if (EPI == kGEpiSoftcap) x = softcap_precise(x, p.cap);
                                obase[(size_t)tok * p.ldo + feat] = from_float<OutT>(x);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
        if (!ok && lane == 0) record_give_up();
    }
    // ---- teardown: everyone is done with tensor memory ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// ---- the same product on pairs of SMs (many tokens) ---------------------------------------------
// Two CTAs of a cluster share one 256 x 256 output tile (tcgen05 cta_group::2): each loads its
// own 128 token rows of A and HALF of the tile's 256 rows of W, the first CTA of the pair issues
// one MMA of M = 256 that reads both CTAs' shared memory, and each CTA's tensor memory receives
// the 128 x 256 accumulator of its own token rows.  Per k-step a CTA stages 32 KB instead of 48
// and the tensor core reads 8 KB of operands per instruction instead of 12, which is what the
// one-CTA kernel is bound by (shared-memory bandwidth: operand reads and TMA writes together).
//
// Who signals whom (all barriers lie at the same offsets in both CTAs):
//   full[s]      the leader's only: its producer expects the bytes of BOTH CTAs' loads; every
//                load names the leader's barrier (address with the pair bit cleared)
//   empty[s]     one per CTA: the leader's commit arrives on both (multicast), so each
//                producer knows when its own stage may be overwritten
//   acc_full[a]  one per CTA, by the leader's multicast commit; each CTA's epilogue waits on its own
//   acc_empty[a] the leader's only: the epilogue warps of both CTAs arrive on it (16 arrivals)
// Tensor memory is allocated and freed by warp 1 of each CTA (the cta_group::2 forms); a
// cluster barrier stands before the first remote arrival and before the release.
struct PairCfg {
    static constexpr int kABytes = GM * GK * 2;             // this CTA's 128 token rows
    static constexpr int kBBytes = 128 * GK * 2;            // this CTA's half of the tile's 256 rows of W
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = 6;
    static constexpr int kStagingBytes = 8 * 4096;          // [32 rows][128 bytes] per epilogue warp
    static constexpr int kSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kStagingBytes;
    static constexpr int kTmemCols = 512;                   // two accumulators of 256 columns
};

template <int EPI, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,     // A: boxes of [128 rows x 64]
                    const __grid_constant__ CUtensorMap map_w,     // W: boxes of [128 rows x 64]
                    GemmParams p) {
    using Cfg = PairCfg;
    constexpr int BN = 256;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~(uintptr_t)1023);
    unsigned char* stages = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + Cfg::kStages;
    uint64_t* acc_full = empty + Cfg::kStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(acc_empty + 2);
    unsigned char* staging = reinterpret_cast<unsigned char*>(bars) + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();               // 0: the leader of the pair
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    const int m_tiles = (p.M + 2 * GM - 1) / (2 * GM);     // tiles of 256 token rows
    constexpr int n_span = EPI == kGEpiGated ? BN / 2 : BN;
    const int n_tiles = (p.N + n_span - 1) / n_span;
    const int k_blocks = (p.K + GK - 1) / GK;
    const int kb_per_split = (k_blocks + p.k_splits - 1) / p.k_splits;      // K may be split over tiles: 32-bit partial sums
    const int total_tiles = m_tiles * n_tiles * p.k_splits;

    if (threadIdx.x == 0) {
        prefetch_tmap(&map_a);
        prefetch_tmap(&map_w);
        for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 16); }
        mbar_fence_init();
    }
    __syncthreads();
    cluster_sync_all();                                    // both CTAs' barriers exist before anything arrives on them
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_smem, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;
    pdl_enter();

    auto tile_coords = [&](int tile, int& mt, int& nt, int& ks) {
        ks = tile % p.k_splits;
        const int t = tile / p.k_splits;
        mt = t % m_tiles;
        nt = t / m_tiles;
    };

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs, each its own halves) ----------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
                int mt, nt, ks;
                tile_coords(tile, mt, nt, ks);
                const int kb0 = ks * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
                const int a_row = mt * 2 * GM + (int)rank * GM;
                const int w_row = EPI == kGEpiGated ? (leader ? nt * 128 : p.gate_rows + nt * 128) : nt * BN + (int)rank * 128;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    if (it >= Cfg::kStages && !mbar_wait_timed(&empty[s], ((it / Cfg::kStages) - 1) & 1)) { ok = false; break; }
                    unsigned char* a_dst = stages + (size_t)s * Cfg::kStageBytes;
                    if (leader) mbar_expect_tx(&full[s], 2 * Cfg::kStageBytes);       // both CTAs' bytes land here
                    tma_load_2d_pair(a_dst, &map_a, kb * GK, a_row, &full[s]);
                    tma_load_2d_pair(a_dst + Cfg::kABytes, &map_w, kb * GK, w_row, &full[s]);
                }
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer: the leader's one thread, for both CTAs ----------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc(2 * GM, BN);
            int it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++local_tile) {
                const int acc = local_tile & 1;
                if (local_tile >= 2 && !mbar_wait_timed(&acc_empty[acc], ((local_tile >> 1) - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int ks = tile % p.k_splits;
                const int kb0 = ks * kb_per_split, kb1 = min(k_blocks, kb0 + kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    if (!mbar_wait_timed(&full[s], (it / Cfg::kStages) & 1)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stages + (size_t)s * Cfg::kStageBytes);
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < GK / 16; ++k)
                        umma_bf16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[acc]);
            }
            if (!ok) record_give_up();
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warps 2..9 of each CTA, its own 128 token rows; warps w and w + 4 share a
        // quarter of the tensor-memory lanes and take half of the tile's columns each ----------------
        const int quarter = warp & 3;
        const int col_half = (warp - 2) >> 2;
        int local_tile = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++local_tile) {
            int mt, nt, ks;
            tile_coords(tile, mt, nt, ks);
            const int acc = local_tile & 1;
            const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            constexpr int COLS = (EPI == kGEpiGated) ? BN / 2 : BN;
            if constexpr (EPI == kGEpiRope) {
                // A tile holds whole heads (head_dim divides 256).  A thread has one token's row of the accumulator;
                // stored, rotated and looked up from there, every access of a warp would touch 32 lines (the table of
                // angles above all: 16 loads of 16 bytes per thread and 32 pairs).  So the warp stages 16 pairs
                // (i, i + head_dim/2) of its 32 rows in shared memory as 32-bit values and finishes them the other
                // way round: four lanes per row, each with four pairs, read the rows' angles line by line, rotate, and
                // store the row to the step's output and, for keys and values, to the cache.
                // While other CTAs stream their operands a load from L2 takes 2 to 3 us, more than a pass's work: what
                // does not depend on the accumulator (the rows' sequences, pages and the angles of the first two
                // passes) is fetched BEFORE the wait for the accumulator, the angles of pass t + 2 right after pass t.
                const RopeEpi& q = p.rope;
                const int hd = q.cache.head_dim, half = hd >> 1;
                unsigned char* stg = staging + (size_t)(warp - 2) * 4096;
                const int m_warp0 = mt * 2 * GM + (int)rank * GM + quarter * 32;
                const int first_head = nt * BN / hd;
                const int heads_in_tile = BN / hd;
                const int sub = lane >> 2, quad = lane & 3;          // second phase: row 8 k + sub, pairs 4 quad .. 4 quad + 3
                // the two warps of a lane quarter share the work: whole heads if the tile holds several, else halves
                // of the one head's pairs
                const int col_begin = heads_in_tile > 1 ? col_half * (BN / 2) : 0, col_end = heads_in_tile > 1 ? col_begin + BN / 2 : BN;
                const int pair_begin = heads_in_tile > 1 ? 0 : col_half * (half / 2), pair_end = heads_in_tile > 1 ? half : pair_begin + half / 2;
                // This lane's four rows of the second phase.  Per row: is it a row of the step, is it rotated (a live
                // sequence), and where its row of the page lies in the cache (kv head 0).
                uint32_t row_mask = 0, rot_mask = 0, cache_mask = 0, rr_low = 0;     // rr_low: (position % 8), four bits a row
                uint32_t cache_row[4];                       // in units of 8 elements (16 bytes): a layer's pages stay far below 2^32 of them
                {
                    int seq4[4], pos4[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int mm = m_warp0 + 8 * k + sub;
                        const bool in_rows = mm < p.M;
                        seq4[k] = in_rows ? q.token_seq[mm] : -1;
                        pos4[k] = in_rows ? q.token_pos[mm] : 0;
                        if (in_rows) row_mask |= 1u << k;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (seq4[k] >= 0) rot_mask |= 1u << k;
                        cache_row[k] = 0;
                        if (seq4[k] >= 0 && q.write_cache && first_head + heads_in_tile > q.n_heads &&
                            !(q.cache.ring_pages > 0 && pos4[k] + q.cache.ring_pages * kPageTokens < q.seq_len_after[seq4[k]])) {
                            const int page = q.cache.page_table[(size_t)q.seq_slot[seq4[k]] * q.cache.table_stride +
                                                                kv_table_entry(q.cache, pos4[k] / kPageTokens)];
                            cache_row[k] = (uint32_t)((kv_tile_offset(q.cache, page, 0) + (size_t)(pos4[k] % kPageTokens) * hd) >> 3);
                            cache_mask |= 1u << k;
                            rr_low |= (uint32_t)(pos4[k] & 7) << (4 * k);
                        }
                    }
                }
                const bool swizzled = kv_is_swizzled(hd);
                const float2* ang_lane = q.angles + (size_t)(m_warp0 + sub) * half + 4 * quad;     // row k: + 8 k half
                auto load_angles = [&](int c0, bool rotated, float4 (&a)[8]) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        a[2 * k] = a[2 * k + 1] = make_float4(1.f, 0.f, 1.f, 0.f);      // values and padding rows are not rotated
                        if (rotated && ((rot_mask >> k) & 1u)) {
                            const float4* src = reinterpret_cast<const float4*>(ang_lane + (size_t)(8 * k) * half + c0);
                            a[2 * k] = __ldg(src);
                            a[2 * k + 1] = __ldg(src + 1);
                        }
                    }
                };
                // the passes of this warp in order: heads outside, 16 pairs inside; (col0, c0) of a pass and of the one
                // two passes on are carried along, not divided out
                int col0 = col_begin, c0 = pair_begin;               // this pass
                int col0_n = col_begin, c0_n = pair_begin;           // the pass whose angles are fetched next
                auto advance = [&](int& cc, int& pc) {
                    pc += 16;
                    if (pc >= pair_end) { pc = pair_begin; cc += hd; }
                };
                auto live = [&](int cc) { return cc < col_end && nt * BN + cc < p.N; };
                auto rotated_head = [&](int cc) { return first_head + cc / hd < q.n_heads + q.n_kv_heads; };
                float4 ang_a[8], ang_b[8];
                if (live(col0_n)) { load_angles(c0_n, rotated_head(col0_n), ang_a); advance(col0_n, c0_n); }
                if (live(col0_n)) { load_angles(c0_n, rotated_head(col0_n), ang_b); advance(col0_n, c0_n); }

                if (!mbar_wait_timed(&acc_full[acc], (local_tile >> 1) & 1)) { ok = false; break; }
                tc_fence_after();
                bf16* out_lane = reinterpret_cast<bf16*>(p.out) + (size_t)(m_warp0 + sub) * p.ldo + nt * BN;   // row k: + 8 k ldo
                const size_t out_step = (size_t)8 * p.ldo;
                // where this lane reads the staged rows: row 8 k + sub has (row & 7) = sub; pieces 2 quad and 2 quad + 1
                const unsigned char* stg_lane = stg + sub * 128;
                const int off0 = ((2 * quad) ^ sub) << 4, off1 = ((2 * quad + 1) ^ sub) << 4;
                bool odd = false;
#pragma unroll 1
                for (; live(col0); advance(col0, c0), odd = !odd) {
                    const int head = first_head + col0 / hd;
                    const bool is_v = head >= q.n_heads + q.n_kv_heads;
                    bf16* pages = nullptr;
                    if (head >= q.n_heads)
                        pages = (bf16*)(is_v ? q.cache.v_pages : q.cache.k_pages) +
                                (size_t)(is_v ? head - q.n_heads - q.n_kv_heads : head - q.n_heads) * kPageTokens * hd;
                    {
                        uint32_t lo[16], hi[16];
                        tmem_ld_32x16(t_lane + col0 + c0, lo);
                        tmem_ld_32x16(t_lane + col0 + half + c0, hi);
                        tmem_ld_wait();
                        unsigned char* srow = stg + lane * 128;
#pragma unroll
                        for (int g = 0; g < 8; ++g)        // piece g: pairs 2g and 2g + 1 as (lo, lo, hi, hi)
                            *reinterpret_cast<uint4*>(srow + ((g ^ (lane & 7)) << 4)) =
                                make_uint4(lo[2 * g], lo[2 * g + 1], hi[2 * g], hi[2 * g + 1]);
                    }
                    __syncwarp();
                    const int col = c0 + 4 * quad;                   // the lane's four low columns; the high ones: + half
                    bf16* out_p = out_lane + col0 + col;
                    const uint32_t cache_mask_here = pages != nullptr ? cache_mask : 0u;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 x0 = *reinterpret_cast<const float4*>(stg_lane + k * 1024 + off0);
                        const float4 x1 = *reinterpret_cast<const float4*>(stg_lane + k * 1024 + off1);
                        const float4 a0 = odd ? ang_b[2 * k] : ang_a[2 * k], a1 = odd ? ang_b[2 * k + 1] : ang_a[2 * k + 1];
                        const uint2 lo4 = make_uint2(pack_bf16(x0.x * a0.x - x0.z * a0.y, x0.y * a0.z - x0.w * a0.w),
                                                     pack_bf16(x1.x * a1.x - x1.z * a1.y, x1.y * a1.z - x1.w * a1.w));
                        const uint2 hi4 = make_uint2(pack_bf16(x0.x * a0.y + x0.z * a0.x, x0.y * a0.w + x0.w * a0.z),
                                                     pack_bf16(x1.x * a1.y + x1.z * a1.x, x1.y * a1.w + x1.w * a1.z));
                        if ((row_mask >> k) & 1u) {
                            *reinterpret_cast<uint2*>(out_p + k * out_step) = lo4;
                            *reinterpret_cast<uint2*>(out_p + k * out_step + half) = hi4;
                        }
                        if ((cache_mask_here >> k) & 1u) {
                            const int rx = swizzled ? (int)((rr_low >> (4 * k)) & 7u) : 0;
                            bf16* crow = pages + ((size_t)cache_row[k] << 3) + (col & 7);
                            *reinterpret_cast<uint2*>(crow + (((col >> 3) ^ rx) << 3)) = lo4;
                            *reinterpret_cast<uint2*>(crow + ((((col + half) >> 3) ^ rx) << 3)) = hi4;
                        }
                    }
                    __syncwarp();
                    if (live(col0_n)) {
                        if (odd) load_angles(c0_n, rotated_head(col0_n), ang_b);
                        else load_angles(c0_n, rotated_head(col0_n), ang_a);
                        advance(col0_n, c0_n);
                    }
                }
            } else {
            if (!mbar_wait_timed(&acc_full[acc], (local_tile >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            // A thread has one token's row of the accumulator, but rows are far apart in memory: stored from here,
            // each 16-byte store of a warp would touch 32 lines.  The warp stages [32 rows][128 bytes] in shared
            // memory (16-byte pieces XOR-permuted by the row, so that neither side conflicts) and copies whole lines
            // out: eight lanes per row, four rows per store.
            constexpr int CW = 128 / (int)sizeof(OutT);            // columns of a staged row
            constexpr int EPP = 16 / (int)sizeof(OutT);            // elements of a 16-byte piece
            unsigned char* stg = staging + (size_t)(warp - 2) * 4096;
            OutT* out_base = reinterpret_cast<OutT*>(p.out) + (p.k_splits > 1 ? (size_t)ks * p.M * p.ldo : 0);
            const int m_warp0 = mt * 2 * GM + (int)rank * GM + quarter * 32;
            const bool vec_ok = (p.ldo % EPP) == 0;
#pragma unroll 1
            for (int c0 = col_half * (COLS / 2); c0 < (col_half + 1) * (COLS / 2); c0 += CW) {
#pragma unroll
                for (int h = 0; h < CW / 32; ++h) {
                    uint32_t v[32], u[32];
                    tmem_ld_32x32(t_lane + c0 + 32 * h, v);
                    if (EPI == kGEpiGated) tmem_ld_32x32(t_lane + BN / 2 + c0 + 32 * h, u);
                    tmem_ld_wait();
                    float f[32];
                    if (EPI == kGEpiGated) {
                        // the kind of activation is tested once, not per element: a select would evaluate both
                        if (p.act == 0) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = gelu_tanh_fast(__uint_as_float(v[j])) * __uint_as_float(u[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = silu_fast(__uint_as_float(v[j])) * __uint_as_float(u[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float x = __uint_as_float(v[j]);
                            f[j] = EPI == kGEpiSoftcap ? softcap_precise(x, p.cap) : x;
                        }
                    }
                    unsigned char* srow = stg + lane * 128;
                    if (sizeof(OutT) == 2) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            *reinterpret_cast<uint4*>(srow + (((4 * h + q) ^ (lane & 7)) << 4)) =
                                make_uint4(pack_bf16(f[8 * q], f[8 * q + 1]), pack_bf16(f[8 * q + 2], f[8 * q + 3]),
                                           pack_bf16(f[8 * q + 4], f[8 * q + 5]), pack_bf16(f[8 * q + 6], f[8 * q + 7]));
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<float4*>(srow + ((q ^ (lane & 7)) << 4)) =
                                make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
                    }
                }
                __syncwarp();
                const int n0 = nt * COLS + c0;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int row = 4 * k + (lane >> 3), piece = lane & 7;
                    const int mm = m_warp0 + row, n = n0 + piece * EPP;
                    const uint4 val = *reinterpret_cast<const uint4*>(stg + row * 128 + ((piece ^ (row & 7)) << 4));
                    if (mm < p.M && n < p.N) {
                        OutT* dst = out_base + (size_t)mm * p.ldo + n;
                        if (vec_ok && n + EPP <= p.N) {
                            *reinterpret_cast<uint4*>(dst) = val;
                        } else {
                            const OutT* e = reinterpret_cast<const OutT*>(&val);
#pragma unroll
                            for (int j = 0; j < EPP; ++j)
                                if (n + j < p.N) dst[j] = e[j];
                        }
                    }
                }
                __syncwarp();
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[acc]);
        }
        if (!ok && lane == 0) record_give_up();
    }
    // ---- teardown: nobody of either CTA touches tensor memory or the other's barriers any more ----
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
}

// Sum K-split partials [splits][M][N] (f32) in a fixed order into out[M][N].
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ part, OutT* __restrict__ out, int M, int N, int ldo,
                                     int splits) {
    pdl_enter();      // the kernels before this one are complete from here on
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * N) return;
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += part[(size_t)k * M * N + i];
    out[(i / N) * ldo + (i % N)] = from_float<OutT>(s);
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// A [rows, K] bf16 matrix with `ld` elements between rows, cut into boxes of [box_rows x 64].
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) HOS_REFUSE("gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)GK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) HOS_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with %d (rows %d K %d ld %d box %d)", (int)r, rows, K, ld, box_rows);
    return 0;
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

template <int BN, int EPI, bool SWAP, typename OutT>
static int launch(const CUtensorMap& mm, const CUtensorMap& mn, const GemmParams& p, int total_tiles, cudaStream_t stream) {
    using Cfg = GemmCfg<BN, SWAP>;
    auto kernel = gemm_tc_kernel<BN, EPI, SWAP, OutT>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem) != cudaSuccess)
            HOS_REFUSE("gemm_tc: cannot get %d bytes of shared memory", Cfg::kSmem);
        attr_set = true;
    }
    const int grid = total_tiles < sm_count() ? total_tiles : sm_count();
    // The gated product of a single-token step (weights as the M operand) follows a norm kernel of a few CTAs:
    // launched ahead of that kernel's end, its barriers and tensor memory are set up meanwhile.  So are the
    // products that leave 32-bit partial sums (q/k/v, o and down of 33 to 128 rows): every kernel here lets its own
    // dependents go only after its wait, so nothing piles up behind them (64 sequences 8.04 -> 7.97 ms a step, 40
    // sequences 5.80 -> 5.75, 128 sequences 14.50 -> 14.44; the head launched ahead changes nothing).
    static const bool swapped_ahead = !(getenv("HOS_GEMM_TC_AHEAD") && getenv("HOS_GEMM_TC_AHEAD")[0] == '0');
    const bool ahead = swapped_ahead && SWAP && (EPI == kGEpiGated || (EPI == kGEpiNone && sizeof(OutT) == 4));
    launch_ahead(pdl_enabled() || ahead, kernel, dim3(grid), dim3(kGemmThreads),
                 Cfg::kSmem, stream, mm, mn, p);
    return check_launch("gemm_tc");
}

// Up to this many rows the weights are the 128-row operand and the tokens the columns (16, 32, 64 or 128 of them).
// It was 64 until the orientations were measured against each other again: a decode step of 72 sequences 9.45 -> 8.95 ms,
// of 128 sequences 14.97 -> 14.46 ms, a prompt of 100 tokens 2.62 -> 2.37 ms (Gemma-2 2B sizes); from 33 to 64 rows the
// kernel on pairs of SMs is 0.7 ms a step slower than this one.
constexpr int kSwapMaxRows = 128;
// From how many rows on a product runs on pairs of SMs: everything above the swapped orientation's rows
// (HOS_GEMM_PAIR=0, or hos_gemm_tc_pair_min_rows(0): never; single SMs with tiles of 128 x 256 run instead).
// It was 512 while the pair kernel's epilogues stored row by row; since they store whole lines a prompt of 70
// to 128 tokens takes 2.7 ms instead of 3.9 (Gemma-2 2B sizes), 129 to 256 tokens 2.9 instead of 4.1, 257 to 384
// 3.4 instead of 4.4, and a decode step of 128 sequences 15.0 ms instead of 15.9.
static int& pair_min_state() {
    static int n = -1;
    if (n < 0) {
        const char* e = getenv("HOS_GEMM_PAIR");
        n = (e && e[0] == '0') ? 0 : kSwapMaxRows + 1;
    }
    return n;
}
static int pair_min_rows() { return pair_min_state(); }
static bool pair_enabled() { return pair_min_state() > 0; }
extern "C" int hos_gemm_tc_pair_min_rows(int rows) {
    if (rows != 0 && rows <= kSwapMaxRows) HOS_REFUSE("gemm_tc: up to %d rows run in the swapped orientation: %d", kSwapMaxRows, rows);
    pair_min_state() = rows;
    return 0;
}

template <int EPI, typename OutT>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, const GemmParams& p, int total_tiles, cudaStream_t stream) {
    auto kernel = gemm_tc_pair_kernel<EPI, OutT>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmem) != cudaSuccess)
            HOS_REFUSE("gemm_tc: cannot get %d bytes of shared memory", PairCfg::kSmem);
        attr_set = true;
    }
    const int pairs_max = sm_count() / 2;
    const int pairs = total_tiles < pairs_max ? total_tiles : pairs_max;
    launch_pdl(kernel, dim3(2 * pairs), dim3(kPairThreads), PairCfg::kSmem, stream, ma, mw, p);
    return check_launch("gemm_tc (pairs of SMs)");
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

// 1 if an earlier launch gave up a bounded wait (and clears the flag).  Synchronises.
extern "C" int hos_gemm_tc_error() {
    int v = 0, zero = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int));
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

// The host's word for waits that ran out (see record_give_up); null takes it away.
extern "C" int hos_gemm_tc_set_error_word(int* word) {
    if (cudaMemcpyToSymbol(g_gemm_error_host, &word, sizeof(word)) != cudaSuccess)
        HOS_REFUSE("gemm_tc: cannot set the error word: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

namespace hos {
// One thread waits, with a limit of `limit_cycles` clock cycles, on a barrier at which nothing ever
// arrives, gives up, records it as the product kernels do, and the kernel ends as usual.
__global__ void wait_probe_kernel(long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        if (!mbar_wait_timed(&bar, 0, limit_cycles)) record_give_up();
    }
}
}  // namespace hos

// For tests of the give-up path: what a product kernel does when a wait runs out, without a product and
// with a short limit (at most 2^24 cycles, a few milliseconds).
extern "C" int hos_gemm_tc_wait_probe(long long limit_cycles, cudaStream_t stream) {
    if (limit_cycles < 1 || limit_cycles > (1ll << 24))
        HOS_REFUSE("gemm_tc_wait_probe: a limit of %lld cycles (1..2^24)", limit_cycles);
    hos::wait_probe_kernel<<<1, 32, 0, stream>>>(limit_cycles);
    return check_launch("gemm_tc_wait_probe");
}

// Floats of workspace for the K-split partial sums of a swapped product (0: no split).
extern "C" long long hos_gemm_tc_workspace(int M, int N, int k_splits) {
    return k_splits > 1 ? (long long)k_splits * M * N : 0;
}

// out[M, N] = A[M, K] . W[N, K]^T, bf16 operands.  out_dtype: 1 bf16, 0 f32.  epilogue: 0 none,
// 1 soft-cap (f32 output), 2 gated (W has 2N rows: gate rows, then up rows at row N).
// M <= 128 runs swapped; k_splits > 1 is allowed only then and only without an epilogue, and
// needs `workspace` (see hos_gemm_tc_workspace).  With reduce_now == 0 the partial sums are left
// in the workspace as [k_splits_used][M][N] floats for the consumer to add, `out` is not written,
// and the number of parts is returned through *parts_used.  lda, ldw, ldo in elements.
extern "C" int hos_gemm_tc(const void* A, const void* W, void* out, int out_dtype, int M, int N, int K, int lda,
                           int ldw, int ldo, int epilogue, float cap, int act, int k_splits, float* workspace,
                           int reduce_now, int* parts_used, cudaStream_t stream) {
    if (parts_used) *parts_used = 1;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) HOS_REFUSE("gemm_tc: K must be positive");
    if ((K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A % 16) || ((uintptr_t)W % 16))
        HOS_REFUSE("gemm_tc: K and the leading dimensions must be multiples of 8 elements and the operands "
                   "16-byte aligned (K %d lda %d ldw %d)", K, lda, ldw);
    if (epilogue == kGEpiSoftcap && out_dtype != kF32) HOS_REFUSE("gemm_tc: the soft-cap epilogue writes 32-bit");
    if (epilogue == kGEpiGated && out_dtype != kBF16) HOS_REFUSE("gemm_tc: the gated epilogue writes bfloat16");
    if (k_splits < 1) k_splits = 1;
    const bool swap = M <= kSwapMaxRows;
    const bool pairs = !swap && M >= pair_min_rows() && pair_enabled();
    if (k_splits > 1 && (!(swap || pairs) || epilogue != kGEpiNone || workspace == nullptr))
        HOS_REFUSE("gemm_tc: K splits need up to %d rows or the kernel on pairs of SMs, no epilogue and a workspace", kSwapMaxRows);
    const int w_rows = epilogue == kGEpiGated ? 2 * N : N;
    GemmParams p;
    p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.k_splits = k_splits; p.gate_rows = N; p.cap = cap; p.act = act;
    CUtensorMap mm, mn;
    const int k_blocks = (K + GK - 1) / GK;
    if (k_splits > k_blocks) k_splits = p.k_splits = k_blocks;
    // no split may be empty: shrink the count until ceil-division leaves none
    while (k_splits > 1 && (k_splits - 1) * ((k_blocks + k_splits - 1) / k_splits) >= k_blocks) k_splits = --p.k_splits;
    int rc;
#define HOS_GO(BN, EPI, SWAP, T, TILES) return launch<BN, EPI, SWAP, T>(mm, mn, p, (TILES), stream)
    if (pairs) {
        // many tokens: tiles of 256 x 256 on pairs of SMs
        if ((rc = make_map(&mm, A, M, K, lda, GM))) return rc;
        if ((rc = make_map(&mn, W, w_rows, K, ldw, 128))) return rc;
        const int m_tiles = (M + 2 * GM - 1) / (2 * GM);
        if (k_splits > 1) {
            // few tiles for the pairs of SMs (a prompt of some hundred tokens): K is split, the partial sums are 32-bit
            p.out = workspace;
            p.ldo = N;
            if ((rc = launch_pair<kGEpiNone, float>(mm, mn, p, m_tiles * ((N + 255) / 256) * k_splits, stream))) return rc;
            if (parts_used) *parts_used = k_splits;
            if (!reduce_now) return 0;
            const size_t n = (size_t)M * N;
            if (out_dtype == kBF16)
                launch_pdl(splitk_reduce_kernel<bf16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, workspace, (bf16*)out, M, N, ldo, k_splits);
            else
                launch_pdl(splitk_reduce_kernel<float>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, workspace, (float*)out, M, N, ldo, k_splits);
            return check_launch("gemm_tc split-K reduce");
        }
        if (epilogue == kGEpiGated) return launch_pair<kGEpiGated, bf16>(mm, mn, p, m_tiles * ((N + 127) / 128), stream);
        const int tiles = m_tiles * ((N + 255) / 256);
        if (epilogue == kGEpiSoftcap) return launch_pair<kGEpiSoftcap, float>(mm, mn, p, tiles, stream);
        if (out_dtype == kBF16) return launch_pair<kGEpiNone, bf16>(mm, mn, p, tiles, stream);
        return launch_pair<kGEpiNone, float>(mm, mn, p, tiles, stream);
    }
    if (!swap) {
        const int m_tiles = (M + GM - 1) / GM;
        constexpr int BN = 256;
        if ((rc = make_map(&mm, A, M, K, lda, GM))) return rc;
        if (epilogue == kGEpiGated) {
            if ((rc = make_map(&mn, W, w_rows, K, ldw, BN / 2))) return rc;
            HOS_GO(256, kGEpiGated, false, bf16, m_tiles * ((N + BN / 2 - 1) / (BN / 2)));
        }
        if ((rc = make_map(&mn, W, w_rows, K, ldw, BN))) return rc;
        const int tiles = m_tiles * ((N + BN - 1) / BN);
        if (epilogue == kGEpiSoftcap) HOS_GO(256, kGEpiSoftcap, false, float, tiles);
        if (out_dtype == kBF16) HOS_GO(256, kGEpiNone, false, bf16, tiles);
        HOS_GO(256, kGEpiNone, false, float, tiles);
    }
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    if ((rc = make_map(&mn, A, M, K, lda, bn))) return rc;
    if (epilogue == kGEpiGated) {
        if ((rc = make_map(&mm, W, w_rows, K, ldw, 64))) return rc;
        const int tiles = (N + 63) / 64;
        if (bn == 16) HOS_GO(16, kGEpiGated, true, bf16, tiles);
        if (bn == 32) HOS_GO(32, kGEpiGated, true, bf16, tiles);
        if (bn == 64) HOS_GO(64, kGEpiGated, true, bf16, tiles);
        HOS_GO(128, kGEpiGated, true, bf16, tiles);
    }
    if ((rc = make_map(&mm, W, w_rows, K, ldw, GM))) return rc;
    const int tiles = ((N + GM - 1) / GM) * k_splits;
    if (k_splits > 1) {
        p.out = workspace;
        p.ldo = N;
        if (bn == 16) rc = launch<16, kGEpiNone, true, float>(mm, mn, p, tiles, stream);
        else if (bn == 32) rc = launch<32, kGEpiNone, true, float>(mm, mn, p, tiles, stream);
        else if (bn == 64) rc = launch<64, kGEpiNone, true, float>(mm, mn, p, tiles, stream);
        else rc = launch<128, kGEpiNone, true, float>(mm, mn, p, tiles, stream);
        if (rc) return rc;
        if (parts_used) *parts_used = k_splits;
        if (!reduce_now) return 0;
        const size_t n = (size_t)M * N;
        if (out_dtype == kBF16)
            launch_pdl(splitk_reduce_kernel<bf16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, workspace, (bf16*)out, M, N, ldo, k_splits);
        else
            launch_pdl(splitk_reduce_kernel<float>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, workspace, (float*)out, M, N, ldo, k_splits);
        return check_launch("gemm_tc split-K reduce");
    }
    if (epilogue == kGEpiSoftcap) {
        if (bn == 16) HOS_GO(16, kGEpiSoftcap, true, float, tiles);
        if (bn == 32) HOS_GO(32, kGEpiSoftcap, true, float, tiles);
        if (bn == 64) HOS_GO(64, kGEpiSoftcap, true, float, tiles);
        HOS_GO(128, kGEpiSoftcap, true, float, tiles);
    }
    if (out_dtype == kBF16) {
        if (bn == 16) HOS_GO(16, kGEpiNone, true, bf16, tiles);
        if (bn == 32) HOS_GO(32, kGEpiNone, true, bf16, tiles);
        if (bn == 64) HOS_GO(64, kGEpiNone, true, bf16, tiles);
        HOS_GO(128, kGEpiNone, true, bf16, tiles);
    }
    if (bn == 16) HOS_GO(16, kGEpiNone, true, float, tiles);
    if (bn == 32) HOS_GO(32, kGEpiNone, true, float, tiles);
    if (bn == 64) HOS_GO(64, kGEpiNone, true, float, tiles);
    HOS_GO(128, kGEpiNone, true, float, tiles);
#undef HOS_GO
}

// The q/k/v projection of many tokens with the rotary encoding and the cache write in its epilogue (pairs of
// SMs): out[M, N] = A . W^T, N = (n_heads + 2 n_kv_heads) * head_dim (n_kv_heads = 0: q heads only), q and k heads
// rotated over the whole head (rotate-half) by the angles[M][head_dim / 2] (cos, sin) of hos_rope_table, keys and
// values stored at the tokens' places if write_cache.
// head_dim 64, 128 or 256; rows enough for the kernel on pairs of SMs; bfloat16 output whose rows are 16-byte aligned.
extern "C" int hos_gemm_tc_qkv_rope(const void* A, const void* W, void* out, int M, int N, int K, int lda, int ldw, int ldo,
                                    int n_heads, int n_kv_heads, int head_dim, const int* token_pos, const int* token_seq,
                                    const int* seq_slot, const int* seq_len_after, const float* angles, void* k_pages,
                                    void* v_pages, const int* page_table, int table_stride, int ring_pages,
                                    int write_cache, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!pair_enabled() || M < pair_min_rows())
        HOS_REFUSE("gemm_tc_qkv_rope: %d rows do not run on pairs of SMs (from %d rows on; 0: never)", M, pair_min_rows());
    if (K <= 0 || (K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A % 16) || ((uintptr_t)W % 16))
        HOS_REFUSE("gemm_tc_qkv_rope: K and the leading dimensions must be multiples of 8 elements and the operands "
                   "16-byte aligned (K %d lda %d ldw %d)", K, lda, ldw);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        HOS_REFUSE("gemm_tc_qkv_rope: head_dim %d is not 64, 128 or 256", head_dim);
    if (n_heads <= 0 || n_kv_heads < 0 || N != (n_heads + 2 * n_kv_heads) * head_dim)
        HOS_REFUSE("gemm_tc_qkv_rope: %d columns are not %d + 2 x %d heads of %d", N, n_heads, n_kv_heads, head_dim);
    if ((ldo % 8) || ((uintptr_t)out % 16)) HOS_REFUSE("gemm_tc_qkv_rope: output rows must be 16-byte aligned");
    if (angles == nullptr || ((uintptr_t)angles % 16) || token_pos == nullptr || token_seq == nullptr)
        HOS_REFUSE("gemm_tc_qkv_rope: positions, sequences and the table of angles (16-byte aligned) are needed");
    if (write_cache && (n_kv_heads == 0 || k_pages == nullptr || v_pages == nullptr || page_table == nullptr ||
                        seq_slot == nullptr || seq_len_after == nullptr))
        HOS_REFUSE("gemm_tc_qkv_rope: the cache write needs kv heads, pages, a page table, slots and lengths");
    GemmParams p;
    p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.k_splits = 1; p.gate_rows = N; p.cap = 0.f; p.act = 0;
    p.rope.token_pos = token_pos; p.rope.token_seq = token_seq; p.rope.seq_slot = seq_slot;
    p.rope.seq_len_after = seq_len_after; p.rope.angles = reinterpret_cast<const float2*>(angles);
    p.rope.cache = PagedKV{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim};
    p.rope.n_heads = n_heads; p.rope.n_kv_heads = n_kv_heads; p.rope.write_cache = write_cache;
    CUtensorMap mm, mn;
    int rc;
    if ((rc = make_map(&mm, A, M, K, lda, GM))) return rc;
    if ((rc = make_map(&mn, W, N, K, ldw, 128))) return rc;
    const int m_tiles = (M + 2 * GM - 1) / (2 * GM);
    return launch_pair<kGEpiRope, bf16>(mm, mn, p, m_tiles * ((N + 255) / 256), stream);
}
