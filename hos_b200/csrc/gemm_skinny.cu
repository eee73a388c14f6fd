// Matrix product for a handful of rows (decoding): out[M, N] = A[M, K] . W[N, K]^T with M <= 32,
// bfloat16 operands, 32-bit accumulation.  The work is reading W once; everything is arranged so
// that nothing stands between the launch and the first bytes of W:
//
//  * no shared-memory staging, no descriptors, no tensor-memory allocation: every thread loads
//    16 bytes of a row of W straight into registers, several loads in flight per thread;
//  * the registers are fed to mma.sync m16n8k16 as they are.  A 16-byte load gives a thread 8
//    consecutive k of one row, while the MMA wants (2t, 2t+1) and (2t+8, 2t+9): since a dot
//    product does not care in which order k is visited, the same permutation of k is applied
//    to both operands (the thread's 16 bytes of an activation row are split the same way), and
//    no shuffle is needed;
//  * a CTA owns 16 output features (rows of W) and its 8 warps split K; their partial tiles
//    are added through shared memory in a fixed order, so no partial sums go through global
//    memory and the result does not depend on timing.
//
// Epilogues: none (bf16 or f32 output); gated, where the CTA owns 16 gate rows and the 16
// matching up rows (4 warps each) and writes act(gate) * up.
#include "common.cuh"
#include "kv_layout.cuh"
#include "mma_utils.cuh"

namespace hos {

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyThreads = kSkinnyWarps * 32;
// A warp walks its share of K in rounds: the loads of U k-blocks of 32 are written before any is used, and a
// round costs a memory latency however few blocks it holds.  So U is chosen (unroll_for, on the host) to deal
// the blocks evenly over the fewest rounds: at K = 2304 a warp has 9 or 18 blocks, which 8 at a time walked in
// 2 or 3 rounds (8 + 1, 8 + 8 + 2) and 9 at a time walks in 1 or 2 (a decode step at 8 sequences 2.243 ->
// 2.19 ms, at 32 sequences 4.75 -> 4.57 ms).  The compiler keeps within 128 registers by issuing some of a
// round's loads between its products; with more than 8 rows more than 9 blocks at a time do not pay.
static int unroll_for(int blocks_per_warp, int token_tiles) {
    const int most = token_tiles == 1 ? 12 : 9;
    const int rounds = (blocks_per_warp + most - 1) / most;
    const int need = rounds > 0 ? (blocks_per_warp + rounds - 1) / rounds : 1;
    if (token_tiles > 1) return need <= 8 ? 8 : 9;
    return need <= 7 ? 7 : (need <= 8 ? 8 : (need <= 9 ? 9 : (need <= 10 ? 10 : 12)));
}
constexpr int kMaxTokenTiles = 4;       // token tiles of 8: up to 32 rows
struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// streaming load for the weights: read once, do not keep in L1
__device__ __forceinline__ uint4 ldg16_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// MT: token tiles of 8 (M <= 8 MT).  GATED: rows come in gate/up pairs.
// WARPS: 8, or 4 for a CTA that keeps half the registers: four such CTAs fit an SM, so a product of up to
// 4 x SMs CTAs runs as ONE wave where CTAs of 8 warps would come in two, with a ramp between them.
template <int MT, int kUnroll, bool GATED, typename OutT, int WARPS = kSkinnyWarps>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS)
gemm_skinny_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, OutT* __restrict__ out,
                   int M, int N, int K, int lda, int ldw, int ldo, int gate_rows, int act, int late) {
    // The kernel may be launched ahead of the end of the kernel before it: its CTAs are placed and a warp's first
    // round of weights, which no kernel writes, is on its way before the activations exist.
    // (`late`: the kernel after this one is let go only when the kernel before this one has ended: this kernel was
    // itself launched ahead, and a chain of kernels that all wait on the SMs costs more than it hides)
    if (!late) pdl_launch_dependents();
    __shared__ float part[WARPS][MT][16][8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int n0 = blockIdx.x * 16;
    // which rows of W this warp reads, and which share of K
    const int k_ways = GATED ? WARPS / 2 : WARPS;
    const int k_way = GATED ? warp % (WARPS / 2) : warp;
    const int row_base = (GATED && warp >= WARPS / 2) ? gate_rows + n0 : n0;
    const int row_limit = (GATED && warp >= WARPS / 2) ? gate_rows + N : N;
    // gridDim.y > 1: K is split over CTAs too; CTA (x, y) writes its 32-bit partial sums to out + y * M * ldo
    const int k_blocks = (K + 31) / 32;
    const int per_cta = (k_blocks + gridDim.y - 1) / gridDim.y;
    const int cta_begin = blockIdx.y * per_cta, cta_end = min(k_blocks, cta_begin + per_cta);
    const int per_way = (max(0, cta_end - cta_begin) + k_ways - 1) / k_ways;
    const int kb_begin = cta_begin + k_way * per_way, kb_end = min(cta_end, kb_begin + per_way);
    out += (size_t)blockIdx.y * M * ldo;

    const int r0 = row_base + g, r1 = row_base + g + 8;
    const bool ok0 = r0 < row_limit, ok1 = r1 < row_limit;
    const bf16* w0 = W + (size_t)(ok0 ? r0 : row_base) * ldw + 8 * t4;
    const bf16* w1 = W + (size_t)(ok1 ? r1 : row_base) * ldw + 8 * t4;
    const bf16* a[MT];
    bool tok[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        a[m] = A + (size_t)min(8 * m + g, M - 1) * lda + 8 * t4;
        tok[m] = 8 * m + g < M;
    }

    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);

    // One round: the loads of kUnroll k-blocks are all written before any is used.  In the first round the
    // weights go out before the wait for the kernel before this one, the activations after it.
    auto round = [&](int kb, auto first) {
        uint4 wa[kUnroll], wb[kUnroll], x[MT][kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k = (kb + u) * 32 + 8 * t4;
            const bool in = (kb + u) < kb_end && k < K;          // K is a multiple of 8: a 16-byte load is whole
            wa[u] = (in && ok0) ? ldg16_stream(w0 + (size_t)(kb + u) * 32) : zero;
            wb[u] = (in && ok1) ? ldg16_stream(w1 + (size_t)(kb + u) * 32) : zero;
            if (!decltype(first)::value) {
#pragma unroll
                for (int m = 0; m < MT; ++m) x[m][u] = (in && tok[m]) ? ldg16(a[m] + (size_t)(kb + u) * 32) : zero;
            }
        }
        if (decltype(first)::value) {
            pdl_wait();       // the kernels before this one are complete from here on: the activations may be read
            if (late) pdl_launch_dependents();
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int k = (kb + u) * 32 + 8 * t4;
                const bool in = (kb + u) < kb_end && k < K;
#pragma unroll
                for (int m = 0; m < MT; ++m) x[m][u] = (in && tok[m]) ? ldg16(a[m] + (size_t)(kb + u) * 32) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            // the thread's 8 consecutive k as two MMAs: k slots (2t,2t+1,2t+8,2t+9) <- elements (0,1,2,3) then (4,5,6,7)
            const uint32_t fa[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            const uint32_t fb[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                mma_bf16(acc[m], fa, x[m][u].x, x[m][u].y);
                mma_bf16(acc[m], fb, x[m][u].z, x[m][u].w);
            }
        }
    };
    if (MT == 1) {
        round(kb_begin, TrueTag{});          // (a warp without a share of K still waits here)
        for (int kb = kb_begin + kUnroll; kb < kb_end; kb += kUnroll) round(kb, FalseTag{});
    } else {
        // more token tiles: the first round is not set apart (its second copy of the loop body costs registers
        // that these shapes do not have: 24 rows 4.06 -> 4.13 ms per step, 32 rows 4.57 -> 4.71 when it was)
        pdl_wait();
        if (late) pdl_launch_dependents();
        for (int kb = kb_begin; kb < kb_end; kb += kUnroll) round(kb, FalseTag{});
    }
    // C fragment: c0 (row g, token 2t), c1 (row g, token 2t+1), c2 (row g+8, token 2t), c3 (row g+8, token 2t+1)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        part[warp][m][g][2 * t4] = acc[m][0];
        part[warp][m][g][2 * t4 + 1] = acc[m][1];
        part[warp][m][g + 8][2 * t4] = acc[m][2];
        part[warp][m][g + 8][2 * t4 + 1] = acc[m][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < MT * 8 * 16; idx += WARPS * 32) {
        const int tok = idx / 16, r = idx % 16;            // consecutive threads: consecutive features of one token
        const int m = tok >> 3, t = tok & 7;
        const int n = n0 + r;
        if (tok >= M || n >= N) continue;
        float v;
        if (GATED) {
            float gsum = 0.f, usum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS / 2; ++w) { gsum += part[w][m][r][t]; usum += part[WARPS / 2 + w][m][r][t]; }
            const float a = act == 0 ? gelu_tanh(gsum) : gsum / (1.f + __expf(-gsum));
            v = a * usum;
        } else {
            v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += part[w][m][r][t];
        }
        out[(size_t)tok * ldo + n] = from_float<OutT>(v);
    }
}


// ---- the q/k/v projection of a decode step with the rotary encoding and the cache write in its
// epilogue ------------------------------------------------------------------------------------
// Same streaming product, but a CTA's 16 rows of W are chosen so that the two rows a rotation pairs
// are rows g and g+8 of the MMA tile: after the K shares are added, one thread holds both values
// of a pair for a token, rotates them (angle = position * inv_freq[i], sincosf in 32-bit), writes
// them to the activation row and, for a key, to the token's place in the paged cache.  Values and
// unrotated dimensions pass straight through.  This saves the separate rotate-and-store launch
// and one round trip of the projection output through memory.
//
// Tiles, in order: for every q head and k head, rot/16 rotation tiles (rotate-half: dims i0..i0+7
// with their partners i0+rot/2..; interleaved: dims 16b..16b+15 as (even, odd)), then (hd-rot)/16
// plain tiles; then hd/16 plain tiles per v head.  Needs head_dim % 16 == 0 and rotary_dim % 16 == 0.
struct QkvRopeArgs {
    const int* token_pos;
    const int* token_seq;
    const int* seq_slot;
    const int* seq_len_after;
    const float* inv_freq;
    PagedKV cache;
    int n_heads, rotary_dim, style, write_cache;
};

template <int MT, int kUnroll>
__global__ void __launch_bounds__(kSkinnyThreads, 2)
qkv_rope_skinny_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, bf16* __restrict__ out,
                       int M, int K, int lda, int ldw, int ldo, QkvRopeArgs q) {
    // The attention kernel after this one may start now: it fetches old keys and values, which this
    // kernel does not touch, and waits for this kernel's end before it reads q or the newest page.
    pdl_launch_dependents();
    __shared__ float part[kSkinnyWarps][MT][16][8 + 1];
    __shared__ int tok_page[MT * 8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int hd = q.cache.head_dim, nkv = q.cache.n_kv_heads, nh = q.n_heads;
    const int rot = q.rotary_dim, half = rot >> 1;
    const int tiles_per_head = hd / 16, rot_tiles = rot / 16;
    // which tile: head (q heads, then k heads, then v heads) and tile within the head
    const int head = blockIdx.x / tiles_per_head, t = blockIdx.x % tiles_per_head;
    const bool is_v = head >= nh + nkv;
    const bool rotated = !is_v && t < rot_tiles;
    // feature (row of W = column of the output) of MMA rows r (0..7) and r+8
    int f_lo, f_hi, step;          // row r -> f_lo + step*r, row r+8 -> f_hi + step*r
    if (rotated && q.style == 0) { f_lo = head * hd + 8 * t; f_hi = f_lo + half; step = 1; }
    else if (rotated) { f_lo = head * hd + 16 * t; f_hi = f_lo + 1; step = 2; }
    else { f_lo = head * hd + 16 * t; f_hi = f_lo + 8; step = 1; }

    const int k_blocks = (K + 31) / 32;
    const int per_way = (k_blocks + kSkinnyWarps - 1) / kSkinnyWarps;
    const int kb_begin = warp * per_way, kb_end = min(k_blocks, kb_begin + per_way);
    const bf16* w0 = W + (size_t)(f_lo + step * g) * ldw + 8 * t4;
    const bf16* w1 = W + (size_t)(f_hi + step * g) * ldw + 8 * t4;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const bf16* a[MT];
    bool tok[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        a[m] = A + (size_t)min(8 * m + g, M - 1) * lda + 8 * t4;
        tok[m] = 8 * m + g < M;
    }
    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    // where each token's key/value goes (looked up while the product runs)
    auto setup_pages = [&]() {
        if (threadIdx.x < MT * 8) {
            int page = -1;
            const int t_ = threadIdx.x;
            if (t_ < M && q.write_cache) {
                const int seq = q.token_seq[t_];
                if (seq >= 0) {
                    const int pos = q.token_pos[t_];
                    if (!(q.cache.ring_pages > 0 && pos + q.cache.ring_pages * kPageTokens < q.seq_len_after[seq]))
                        page = q.cache.page_table[(size_t)q.seq_slot[seq] * q.cache.table_stride +
                                                  kv_table_entry(q.cache, pos / kPageTokens)];
                }
            }
            tok_page[t_] = page;
        }
    };
    auto round = [&](int kb) {
        uint4 wa[kUnroll], wb[kUnroll], x[MT][kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k = (kb + u) * 32 + 8 * t4;
            const bool in = (kb + u) < kb_end && k < K;
            wa[u] = in ? ldg16_stream(w0 + (size_t)(kb + u) * 32) : zero;
            wb[u] = in ? ldg16_stream(w1 + (size_t)(kb + u) * 32) : zero;
#pragma unroll
            for (int m = 0; m < MT; ++m) x[m][u] = (in && tok[m]) ? ldg16(a[m] + (size_t)(kb + u) * 32) : zero;
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t fa[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            const uint32_t fb[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                mma_bf16(acc[m], fa, x[m][u].x, x[m][u].y);
                mma_bf16(acc[m], fb, x[m][u].z, x[m][u].w);
            }
        }
    };
    pdl_wait();               // the kernels before this one are complete from here on
    setup_pages();
    for (int kb = kb_begin; kb < kb_end; kb += kUnroll) round(kb);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        part[warp][m][g][2 * t4] = acc[m][0];
        part[warp][m][g][2 * t4 + 1] = acc[m][1];
        part[warp][m][g + 8][2 * t4] = acc[m][2];
        part[warp][m][g + 8][2 * t4 + 1] = acc[m][3];
    }
    __syncthreads();
    // one thread per (token, pair): rows r and r+8 of the tile
    for (int idx = threadIdx.x; idx < MT * 8 * 8; idx += kSkinnyThreads) {
        const int tok = idx / 8, r = idx % 8;
        if (tok >= M) continue;
        const int m = tok >> 3, tt = tok & 7;
        float v0 = 0.f, v1 = 0.f;
#pragma unroll
        for (int w = 0; w < kSkinnyWarps; ++w) { v0 += part[w][m][r][tt]; v1 += part[w][m][r + 8][tt]; }
        const int seq = q.token_seq[tok];
        if (seq < 0) continue;                                   // padding: nothing is stored
        const int fa_ = f_lo + step * r, fb_ = f_hi + step * r;
        if (rotated) {
            const int i = 8 * t + r;                             // index of the pair within the head
            float sn, cs;
            sincosf((float)q.token_pos[tok] * q.inv_freq[i], &sn, &cs);
            const float x0 = v0, x1 = v1;
            v0 = x0 * cs - x1 * sn;
            v1 = x0 * sn + x1 * cs;
        }
        const bf16 b0 = __float2bfloat16_rn(v0), b1 = __float2bfloat16_rn(v1);
        out[(size_t)tok * ldo + fa_] = b0;
        out[(size_t)tok * ldo + fb_] = b1;
        const int page = tok_page[tok];
        if (head >= nh && page >= 0) {                          // a key or a value: into the cache
            const int kvh = is_v ? head - nh - nkv : head - nh;
            bf16* base = (bf16*)(is_v ? q.cache.v_pages : q.cache.k_pages) + kv_tile_offset(q.cache, page, kvh);
            const int rr = q.token_pos[tok] % kPageTokens;
            base[kv_elem_offset(rr, fa_ - head * hd, hd)] = b0;
            base[kv_elem_offset(rr, fb_ - head * hd, hd)] = b1;
        }
    }
}

}  // namespace hos

using namespace hos;

extern "C" const char* hos_last_error() { return error_buffer(); }

// Whether the few-rows products are launched ahead of the end of the kernel before them (their first weights
// are then fetched while that kernel finishes): HOS_SKINNY_AHEAD=0 or 1 in the environment.
// Which few-rows products are launched ahead of the end of the kernel before them.  Of up to 8 rows: bits 1 gate/up,
// 2 products with bfloat16 output (o), 4 products that write partial sums (down), 8 the q/k/v projection; of 9 to 32
// rows (without weights fetched early): 16 gate/up, 32 the q/k/v projection.  HOS_SKINNY_AHEAD in the environment,
// default 57 (see below).
static int skinny_ahead_mode() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("HOS_SKINNY_AHEAD");
        on = (e && e[0]) ? atoi(e) : 61;
    }
    return on;
}
static bool skinny_ahead(int kind) { return (skinny_ahead_mode() & kind) != 0 || pdl_enabled(); }
// The gate/up product and the q/k/v projection of a step of up to 8 rows each follow a norm kernel of 8 CTAs:
// launched ahead of that kernel's end, their CTAs are placed and (gate/up) their first weights on their way while
// the norm runs.  Measured on a batch-8 step of Gemma-2 2B sizes (ms per step; one sequence in brackets): none
// ahead 2.123 (1.502), gate/up 2.118 (1.500), gate/up and q/k/v 2.111 (1.495), gate/up and down 2.125 (1.497),
// gate/up and o 2.414 (1.598), all four 2.697 (1.790).  The o and down products follow kernels that fill the SMs
// (and the attention before o is itself launched ahead of q/k/v): launched ahead they take places too early.
// With 9 to 32 rows the two products behind a norm are launched ahead as well, only to have their CTAs placed (12 rows
// 2.652 -> 2.625 ms, 16 rows 2.958 -> 2.936, 32 rows 4.564 -> 4.558).
// What cost the down product its place in that list was the chain behind it: launched ahead, it let the norm after it
// go at once, which let the q/k/v projection go, and all of them sat waiting on the SMs.  Launched ahead but letting
// its own dependents go only when the kernel before it has ended (`late`), it gains: a step of 8 sequences 2.128 ->
// 2.101 ms, one sequence 1.478 -> 1.464, 2 sequences 1.585 -> 1.562, 8 sequences at 1,024 keys 1.487 -> 1.464.  The o
// product the same way gains 3% for one sequence up to 8,192 keys (1.478 -> 1.436 ms with both) and loses 7 to 20%
// everywhere else (2, 4 or 8 sequences; one sequence at 32,768 keys): it stays behind its attention kernel.

// out[M, N] = A[M, K] . W[N, K]^T for M <= 32.  epilogue 0: none (out bf16 or f32); 2: gated (W has
// 2N rows: gate rows, then up rows at row N; out bf16).  K and the leading dimensions must be
// multiples of 8 elements, A and W 16-byte aligned.
// k_splits > 1: `out` is [k_splits][M][ldo] 32-bit partial sums for a consumer that adds them (no epilogue).
extern "C" int hos_gemm_skinny(const void* A, const void* W, void* out, int out_dtype, int M, int N, int K,
                               int lda, int ldw, int ldo, int epilogue, int act, int k_splits, int room_before,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 8 * kMaxTokenTiles) HOS_REFUSE("gemm_skinny: %d rows are more than %d", M, 8 * kMaxTokenTiles);
    if (K <= 0 || (K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A % 16) || ((uintptr_t)W % 16))
        HOS_REFUSE("gemm_skinny: K and the leading dimensions must be multiples of 8 elements and the operands "
                   "16-byte aligned (K %d lda %d ldw %d)", K, lda, ldw);
    if (epilogue != 0 && epilogue != 2) HOS_REFUSE("gemm_skinny: epilogue %d is not offered", epilogue);
    if (epilogue == 2 && out_dtype != kBF16) HOS_REFUSE("gemm_skinny: the gated epilogue writes bfloat16");
    if (k_splits < 1 || k_splits > 64) HOS_REFUSE("gemm_skinny: %d splits of K (1..64)", k_splits);
    if (k_splits > 1 && (epilogue != 0 || out_dtype != kF32))
        HOS_REFUSE("gemm_skinny: partial sums over a split K are 32-bit and take no epilogue");
    const unsigned grid = (unsigned)((N + 15) / 16);
    // The gated product has the most CTAs (gate/up of a feed-forward): with 4 warps each, four of them fit an SM
    // and the waves are half as many (Gemma-2 2B sizes: 576 CTAs are one wave instead of two; a batch-8 step
    // 2.137 -> 2.126 ms, one sequence 1.505 -> 1.498, 32 sequences 4.66 -> 4.63).
    constexpr int kGatedWarps = 4;
    const int k_ways = epilogue == 2 ? kGatedWarps / 2 : kSkinnyWarps;
    const int k_blocks = (K + 31) / 32, per_cta = (k_blocks + k_splits - 1) / k_splits;
    const int unroll = unroll_for((per_cta + k_ways - 1) / k_ways, (M + 7) / 8);
    const int kind = (M > 8) ? (epilogue == 2 ? 16 : 0) : (epilogue == 2 ? 1 : (out_dtype == kBF16 ? 2 : 4));
    // `room_before` (the caller's word that the kernel before this one leaves at least half of the SMs free, as the
    // attention of one sequence does): the o product is then launched ahead as well
    const bool ahead = skinny_ahead(kind) || (kind == 2 && room_before != 0);
    const int late = (kind == 2 || kind == 4) && ahead ? 1 : 0;     // o and down, when launched ahead
#define HOS_SK_W(MT, U, G, T, WP)                                                                                \
    launch_ahead(ahead, gemm_skinny_kernel<MT, U, G, T, WP>, dim3(grid, k_splits), dim3(WP * 32), 0, stream, (const bf16*)A, (const bf16*)W, (T*)out, \
                                                                       M, N, K, lda, ldw, ldo, N, act, late)
#define HOS_SK(MT, U, G, T) HOS_SK_W(MT, U, G, T, (G ? kGatedWarps : kSkinnyWarps))
#define HOS_SK_U(MT, G, T)                              \
    do {                                                \
        if (unroll == 8) HOS_SK(MT, 8, G, T);           \
        else HOS_SK(MT, 9, G, T);                       \
    } while (0)
#define HOS_SK_M(G, T)                                  \
    do {                                                \
        if (M <= 8) {                                   \
            if (unroll == 7) HOS_SK(1, 7, G, T);        \
            else if (unroll == 8) HOS_SK(1, 8, G, T);   \
            else if (unroll == 9) HOS_SK(1, 9, G, T);   \
            else if (unroll == 10) HOS_SK(1, 10, G, T); \
            else HOS_SK(1, 12, G, T);                   \
        } else if (M <= 16) HOS_SK_U(2, G, T);          \
        else if (M <= 24) HOS_SK_U(3, G, T);            \
        else HOS_SK_U(4, G, T);                         \
    } while (0)
    if (epilogue == 2) {
        HOS_SK_M(true, bf16);
    } else if (out_dtype == kBF16) {
        HOS_SK_M(false, bf16);
    } else if (out_dtype == kF32) {
        HOS_SK_M(false, float);
    } else {
        HOS_REFUSE("gemm_skinny: unknown output dtype %d", out_dtype);
    }
#undef HOS_SK_U
#undef HOS_SK_M
#undef HOS_SK
#undef HOS_SK_W
    return check_launch("gemm_skinny");
}

// The q/k/v projection of up to 32 tokens with rotary encoding and cache write fused in:
// out[M, (n_heads + 2 n_kv_heads) * head_dim] = A[M, K] . W^T, q and k heads rotated, keys and values
// stored at the tokens' places.  Needs head_dim % 16 == 0 and rotary_dim % 16 == 0 (0: no rotation).
extern "C" int hos_qkv_rope_skinny(const void* A, const void* W, void* out, int M, int K, int lda, int ldw, int ldo,
                                   int n_heads, int n_kv_heads, int head_dim, const int* token_pos,
                                   const int* token_seq, const int* seq_slot, const int* seq_len_after,
                                   const float* inv_freq, int rotary_dim, int style, void* k_pages, void* v_pages,
                                   const int* page_table, int table_stride, int ring_pages, int write_cache,
                                   cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 8 * kMaxTokenTiles) HOS_REFUSE("qkv_rope_skinny: %d rows are more than %d", M, 8 * kMaxTokenTiles);
    if (K <= 0 || (K % 8) || (lda % 8) || (ldw % 8) || ((uintptr_t)A % 16) || ((uintptr_t)W % 16))
        HOS_REFUSE("qkv_rope_skinny: K and the leading dimensions must be multiples of 8 elements and the operands "
                   "16-byte aligned (K %d lda %d ldw %d)", K, lda, ldw);
    if ((head_dim % 16) || (rotary_dim % 16) || rotary_dim < 0 || rotary_dim > head_dim || (style != 0 && style != 1))
        HOS_REFUSE("qkv_rope_skinny: head_dim %d and rotary_dim %d must be multiples of 16", head_dim, rotary_dim);
    QkvRopeArgs q;
    q.token_pos = token_pos; q.token_seq = token_seq; q.seq_slot = seq_slot; q.seq_len_after = seq_len_after;
    q.inv_freq = inv_freq;
    q.cache = PagedKV{k_pages, v_pages, page_table, table_stride, ring_pages, n_kv_heads, head_dim};
    q.n_heads = n_heads; q.rotary_dim = rotary_dim; q.style = style; q.write_cache = write_cache;
    const unsigned grid = (unsigned)((n_heads + 2 * n_kv_heads) * (head_dim / 16));
    const int unroll = unroll_for(((K + 31) / 32 + kSkinnyWarps - 1) / kSkinnyWarps, (M + 7) / 8);
#define HOS_QR(MT, U)                                                                                                      \
    launch_ahead(skinny_ahead(MT == 1 ? 8 : 32), qkv_rope_skinny_kernel<MT, U>, dim3(grid), dim3(kSkinnyThreads), 0, stream, (const bf16*)A, (const bf16*)W, \
               (bf16*)out, M, K, lda, ldw, ldo, q)
#define HOS_QR_U(MT)                     \
    do {                                 \
        if (unroll == 8) HOS_QR(MT, 8);  \
        else HOS_QR(MT, 9);              \
    } while (0)
    if (M <= 8) {
        if (unroll == 7) HOS_QR(1, 7);
        else if (unroll == 8) HOS_QR(1, 8);
        else if (unroll == 9) HOS_QR(1, 9);
        else if (unroll == 10) HOS_QR(1, 10);
        else HOS_QR(1, 12);
    } else if (M <= 16) HOS_QR_U(2);
    else if (M <= 24) HOS_QR_U(3);
    else HOS_QR_U(4);
#undef HOS_QR_U
#undef HOS_QR
    return check_launch("qkv_rope_skinny");
}
