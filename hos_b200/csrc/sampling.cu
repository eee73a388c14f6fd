// Token choice on the device, one block per sequence.  The order of operations is
// the reference sampler's (src/lib.rs:91-172): repetition penalty over the recent
// tokens (once per occurrence, :102-118); temp <= 0 -> arg max, first maximum wins
// (:120-128); else p_i = exp((l_i - max) / temp) (:130-135); keep the top_k most
// probable (:142-148), then the shortest prefix of them, in falling order of
// probability, whose mass reaches top_p (:149-160); draw r = u * (kept mass) and walk
// the kept tokens in that same order until the running sum exceeds r (:162-171).
// u comes from the caller's xorshift64 stream (src/lib.rs:78-85).
//
// The reference sorts; this kernel never does.  Everything above depends only on the
// order "higher probability first, lower token id first among equals", so the k-th
// token, the top_p cut and the drawn token are found by radix selection: per pass a
// histogram (of counts or of probability mass) over one digit of an order-preserving
// integer image of the logit, kept private per thread in shared memory so that no
// atomics are needed, then a walk over the 32 bins.  Equal logits have equal
// probability, so positions among equals follow by division and a selection on the id.
#include "common.cuh"

namespace hos {

constexpr int kThreads = 512;
constexpr int kDigitBits = 5;
constexpr int kBins = 1 << kDigitBits;
constexpr int kScanUnroll = 8;
constexpr int kSmallSet = 1024;       // kept sets up to this size are sorted in shared memory, as the reference sorts

__device__ __forceinline__ uint32_t order_key(float v) {
    uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float -> larger key
}

struct Kept {          // the kept set: key > x, or key == x and id <= last_id
    uint32_t x;
    int last_id;
};
__device__ __forceinline__ bool in_kept(const Kept& k, uint32_t key, int id) {
    return key > k.x || (key == k.x && id <= k.last_id);
}

struct SelectResult {
    bool found;
    uint32_t x;        // the selected digit string
    float above;       // weight of everything ordered before it
    float equal;       // weight of the elements that share it
};

// Radix selection, most significant digit first, over elements for which `filter`
// holds, ordered by `keyfn` descending, with weights `wfn`.  Finds x with
//   strict == false:  W(key > x) <  target <= W(key >= x)
//   strict == true :  W(key > x) <= target <  W(key >= x)
// hist: kBins * kThreads floats of shared memory; red: kBins floats.
template <typename KeyFn, typename WFn, typename FilterFn>
__device__ SelectResult radix_select(int V, int nbits, float target, bool strict, KeyFn keyfn,
                                     WFn wfn, FilterFn filter, float* hist, float* red) {
    const int tid = threadIdx.x;
    uint32_t prefix = 0, prefix_mask = 0;
    float above = 0.f, equal = 0.f;
    const int passes = (nbits + kDigitBits - 1) / kDigitBits;
    for (int pass = 0; pass < passes; ++pass) {
        const int shift = max(0, nbits - (pass + 1) * kDigitBits);
        const int width = min(kDigitBits, nbits - pass * kDigitBits);
        const uint32_t dmask = (1u << width) - 1u;
        for (int b = 0; b < kBins; ++b) hist[b * kThreads + tid] = 0.f;
        for (int i0 = tid; i0 < V; i0 += kThreads * kScanUnroll) {        // several loads in flight per thread
            uint32_t key[kScanUnroll];
            bool take[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) {
                const int i = i0 + u * kThreads;
                take[u] = i < V && filter(i);
                key[u] = take[u] ? keyfn(i) : 0u;
            }
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u)
                if (take[u] && (key[u] & prefix_mask) == prefix)       // the weight only of what is still in the running
                    hist[((key[u] >> shift) & dmask) * kThreads + tid] += wfn(i0 + u * kThreads);
        }
        __syncthreads();
        // reduce each bin over the threads: 16 threads per bin, 32 columns each
        {
            const int bin = tid >> 4, part = tid & 15;
            float s = 0.f;
            for (int c = part; c < kThreads; c += 16) s += hist[bin * kThreads + c];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (part == 0) red[bin] = s;
        }
        __syncthreads();
        // every thread walks the bins from the highest digit down (same result everywhere)
        int chosen = -1, lowest = -1;
        float acc = above, acc_lowest = above;
        for (int b = (int)dmask; b >= 0; --b) {
            const float next = acc + red[b];
            const bool cross = strict ? (next > target) : (next >= target);
            if (red[b] > 0.f) { lowest = b; acc_lowest = acc; }
            if (cross && red[b] > 0.f) { chosen = b; break; }
            acc = next;
        }
        __syncthreads();
        if (chosen < 0 && pass > 0 && lowest >= 0) {
            // the parent bin crossed the target but, summed in another order, its parts
            // fall a rounding short: the crossing is in the last non-empty part
            chosen = lowest;
            acc = acc_lowest;
        }
        if (chosen < 0) return SelectResult{false, 0u, acc, 0.f};
        above = acc;
        equal = red[chosen];
        prefix |= ((uint32_t)chosen) << shift;
        prefix_mask |= dmask << shift;
        __syncthreads();
    }
    return SelectResult{true, prefix, above, equal};
}

// id of the j-th (1-based) smallest token id among kept elements whose key is x
template <typename KeyFn>
__device__ int nth_equal_id(int V, uint32_t x, const Kept& kept, int j, int id_bits, KeyFn keyfn,
                            float* hist, float* red) {
    const uint32_t idmask = (1u << id_bits) - 1u;
    SelectResult r = radix_select(
        V, id_bits, (float)j, false,
        [&](int i) { return (~(uint32_t)i) & idmask; },      // descending in ~id = ascending in id
        [&](int) { return 1.f; },
        [&](int i) { return keyfn(i) == x && in_kept(kept, x, i); }, hist, red);
    if (!r.found) return -1;
    return (int)((~r.x) & idmask);
}

// One scan: how many kept elements have key x, and the lowest and highest id among them.  With
// these the j-th of them is known at once when it is the first or the last (the common cases: a
// key that occurs once, or all of the equals wanted); only otherwise is a selection on the id run.
struct EqualInfo { int n, min_id, max_id; };
template <typename KeyFn>
__device__ EqualInfo equal_scan(int V, uint32_t x, const Kept& kept, KeyFn keyfn, int* sh3) {
    int n = 0, lo = 0x7fffffff, hi = -1;
    for (int i0 = threadIdx.x; i0 < V; i0 += kThreads * kScanUnroll) {
        uint32_t key[kScanUnroll];
#pragma unroll
        for (int u = 0; u < kScanUnroll; ++u) key[u] = (i0 + u * kThreads) < V ? keyfn(i0 + u * kThreads) : 0u;
#pragma unroll
        for (int u = 0; u < kScanUnroll; ++u) {
            const int i = i0 + u * kThreads;
            if (i < V && key[u] == x && in_kept(kept, x, i)) { ++n; lo = min(lo, i); hi = max(hi, i); }
        }
    }
    if (threadIdx.x == 0) { sh3[0] = 0; sh3[1] = 0x7fffffff; sh3[2] = -1; }
    __syncthreads();
    if (n) { atomicAdd(&sh3[0], n); atomicMin(&sh3[1], lo); atomicMax(&sh3[2], hi); }     // integers: order does not matter
    __syncthreads();
    EqualInfo e{sh3[0], sh3[1], sh3[2]};
    __syncthreads();
    return e;
}
template <typename KeyFn>
__device__ int jth_equal(int V, uint32_t x, const Kept& kept, int j, const EqualInfo& e, int id_bits, KeyFn keyfn,
                         float* hist, float* red) {
    if (j <= 1) return e.min_id;
    if (j >= e.n) return e.max_id;
    return nth_equal_id(V, x, kept, j, id_bits, keyfn, hist, red);
}
__device__ __forceinline__ float value_of_key(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// One block per row.  logits rows are modified in place for the penalty and restored.
__global__ void __launch_bounds__(kThreads)
sample_kernel(float* __restrict__ logits, int ld, int V, const float* __restrict__ uniforms,
              const int* __restrict__ recent, int recent_stride, const int* __restrict__ recent_len,
              float temp, int top_k, float top_p, float rep_penalty, int* __restrict__ out) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ float smem[];
    float* hist = smem;                       // kBins * kThreads
    float* red = hist + kBins * kThreads;     // kBins
    float* scratch = red + kBins;             // 32
    __shared__ float saved_val[256];
    __shared__ int saved_id[256];
    __shared__ int n_saved;
    __shared__ int best_id_sh;
    __shared__ int eq_sh[3];
    const int row = blockIdx.x, tid = threadIdx.x;
    float* l = logits + (size_t)row * ld;

    // repetition penalty, once per occurrence, first-seen originals remembered
    const int nrec = (recent != nullptr && rep_penalty != 1.0f) ? min(recent_len[row], 256) : 0;
    if (tid == 0) {
        int ns = 0;
        for (int j = 0; j < nrec; ++j) {
            const int t = recent[(size_t)row * recent_stride + j];
            if (t < 0 || t >= V) continue;
            bool seen = false;
            for (int s = 0; s < ns; ++s) seen |= (saved_id[s] == t);
            if (!seen) { saved_id[ns] = t; saved_val[ns] = l[t]; ++ns; }
            const float v = l[t];
            l[t] = v > 0.f ? v / rep_penalty : v * rep_penalty;
        }
        n_saved = ns;
        __threadfence_block();
    }
    __syncthreads();

    int result;
    // ---- arg max (also needed for the softmax's maximum) ----
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += kThreads) {
        const float v = l[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    const float maxv = block_max(best, scratch);
    {
        // lowest id among the threads that hold the maximum
        int cand = (best == maxv) ? best_i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __shared__ int warp_best[kThreads / 32];
        if ((tid & 31) == 0) warp_best[tid >> 5] = cand;
        __syncthreads();
        if (tid == 0) {
            int b = 0x7fffffff;
            for (int w = 0; w < kThreads / 32; ++w) b = min(b, warp_best[w]);
            best_id_sh = b;
        }
        __syncthreads();
    }
    if (temp <= 0.f) {
        result = best_id_sh;
    } else {
        auto keyfn = [&](int i) { return order_key(l[i]); };
        auto prob = [&](int i) { return expf((l[i] - maxv) / temp); };   // not normalised
        int id_bits = 1;
        while ((1 << id_bits) < V) ++id_bits;
        float z = 0.f;
        for (int i0 = tid; i0 < V; i0 += kThreads * kScanUnroll) {
            float v[kScanUnroll];
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) v[u] = (i0 + u * kThreads) < V ? l[i0 + u * kThreads] : -INFINITY;
#pragma unroll
            for (int u = 0; u < kScanUnroll; ++u) z += expf((v[u] - maxv) / temp);      // exp(-inf) = 0 beyond the end
        }
        z = block_sum(z, scratch);

        Kept kept{0u, V};      // everything
        float kept_mass = z;
        bool small_done = false;
        auto all = [&](int) { return true; };
        auto kept_filter = [&](int i) { return in_kept(kept, keyfn(i), i); };
        // ---- top-k ----
        if (top_k > 0 && top_k < V) {
            SelectResult r = radix_select(V, 32, (float)top_k, false, keyfn,
                                          [&](int) { return 1.f; }, all, hist, red);
            // r.found always holds here: top_k < V elements exist
            const int need = top_k - (int)r.above;          // how many of the equals stay
            Kept whole{r.x, V};
            const EqualInfo eq = equal_scan(V, r.x, whole, keyfn, eq_sh);
            const int last = jth_equal(V, r.x, whole, need, eq, id_bits, keyfn, hist, red);
            kept = Kept{r.x, last};
            if (top_k <= kSmallSet) {
                // The kept tokens fit shared memory: gather them, sort them (probability falling, id
                // rising among equals) and let one thread do what the reference does on its sorted list.
                __shared__ unsigned long long cand[kSmallSet];
                __shared__ int n_cand;
                if (tid == 0) n_cand = 0;
                __syncthreads();
                for (int i0 = tid; i0 < V; i0 += kThreads * kScanUnroll) {
                    float v[kScanUnroll];
#pragma unroll
                    for (int u = 0; u < kScanUnroll; ++u) v[u] = (i0 + u * kThreads) < V ? l[i0 + u * kThreads] : 0.f;
#pragma unroll
                    for (int u = 0; u < kScanUnroll; ++u) {
                        const int i = i0 + u * kThreads;
                        if (i < V && in_kept(kept, order_key(v[u]), i)) {
                            const int at = atomicAdd(&n_cand, 1);
                            if (at < kSmallSet)
                                cand[at] = ((unsigned long long)order_key(v[u]) << 32) | (uint32_t)(~(uint32_t)i);
                        }
                    }
                }
                __syncthreads();
                const int n = min(n_cand, kSmallSet);
                int n2 = 1;
                while (n2 < n) n2 <<= 1;
                for (int i = n + tid; i < n2; i += kThreads) cand[i] = 0ull;        // padding sorts last
                __syncthreads();
                for (int k = 2; k <= n2; k <<= 1)                                   // bitonic sort, descending
                    for (int j = k >> 1; j > 0; j >>= 1) {
                        for (int i = tid; i < n2; i += kThreads) {
                            const int ixj = i ^ j;
                            if (ixj > i) {
                                const unsigned long long a = cand[i], b = cand[ixj];
                                const bool desc = (i & k) == 0;
                                if (desc ? (a < b) : (a > b)) { cand[i] = b; cand[ixj] = a; }
                            }
                        }
                        __syncthreads();
                    }
                if (tid == 0) {
                    auto value_of = [](unsigned long long c) {
                        const uint32_t key = (uint32_t)(c >> 32);
                        return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
                    };
                    auto prob_of = [&](unsigned long long c) { return expf((value_of(c) - maxv) / temp) / z; };
                    int cut = n;
                    if (top_p < 1.0f) {
                        float cum = 0.f;
                        for (int i = 0; i < n; ++i) {
                            cum += prob_of(cand[i]);
                            if (cum >= top_p) { cut = i + 1; break; }
                        }
                    }
                    float total = 0.f;
                    for (int i = 0; i < cut; ++i) total += prob_of(cand[i]);
                    const float rr = uniforms[row] * total;
                    float cdf = 0.f;
                    int pick = cut - 1;
                    for (int i = 0; i < cut; ++i) {
                        cdf += prob_of(cand[i]);
                        if (rr < cdf) { pick = i; break; }
                    }
                    best_id_sh = (int)(~(uint32_t)(cand[pick] & 0xffffffffull));
                }
                __syncthreads();
                result = best_id_sh;
                small_done = true;
            } else {
                float m = 0.f;
                for (int i = tid; i < V; i += kThreads)
                    if (kept_filter(i)) m += prob(i);
                kept_mass = block_sum(m, scratch);
            }
        }
        if (!small_done) {
        // ---- top-p: shortest prefix whose mass reaches top_p of the WHOLE distribution ----
        if (top_p < 1.0f) {
            const float target = top_p * z;
            SelectResult r = radix_select(V, 32, target, false, keyfn, prob, kept_filter, hist, red);
            if (r.found) {
                // equals share one probability; the prefix needs j of them
                const EqualInfo eq = equal_scan(V, r.x, kept, keyfn, eq_sh);
                const int n_eq = eq.n;
                const float p_eq = expf((value_of_key(r.x) - maxv) / temp);
                int j = (int)ceilf((target - r.above) / p_eq);
                j = max(1, min(j, n_eq));
                const int last = jth_equal(V, r.x, kept, j, eq, id_bits, keyfn, hist, red);
                kept = Kept{r.x, last};
                kept_mass = r.above + (float)j * p_eq;
            }
        }
        // ---- draw ----
        const float rr = uniforms[row] * kept_mass;
        SelectResult r = radix_select(V, 32, rr, true, keyfn, prob, kept_filter, hist, red);
        if (!r.found) {
            result = kept.last_id < V ? kept.last_id : -1;
            if (result < 0) {
                // the kept set is everything: its last element is the least probable, highest id
                SelectResult lo = radix_select(V, 32, (float)V, false, keyfn,
                                               [&](int) { return 1.f; }, all, hist, red);
                int n_eq = (int)(lo.equal + 0.5f);
                Kept whole{lo.x, V};
                result = nth_equal_id(V, lo.x, whole, n_eq, id_bits, keyfn, hist, red);
            }
        } else {
            const EqualInfo eq = equal_scan(V, r.x, kept, keyfn, eq_sh);
            const int n_eq = eq.n;
            const float p_eq = expf((value_of_key(r.x) - maxv) / temp);
            int j = (int)floorf((rr - r.above) / p_eq) + 1;
            j = max(1, min(j, n_eq));
            result = jth_equal(V, r.x, kept, j, eq, id_bits, keyfn, hist, red);
        }
        }   // !small_done
    }
    __syncthreads();
    if (tid == 0) {
        for (int s = 0; s < n_saved; ++s) l[saved_id[s]] = saved_val[s];
        out[row] = result;
    }
}

// ---- the same choice by a cluster of 8 CTAs per row, for temp > 0 and 1 <= top_k <= 1024 ----------
// A CTA keeps an eighth of the row in its shared memory (read from global memory once, the
// repetition penalty applied to the copy), so every later pass runs on shared memory; what the
// CTAs have to agree on (maximum, normaliser, the histograms of the radix selection of the
// top_k-th key, how many of its equals each holds) goes through distributed shared memory and a
// cluster barrier.  The kept tokens are gathered into the first CTA, which sorts them
// (probability falling, id rising among equals) and walks them as the reference walks its list.
// Every CTA takes the same branches, so every cluster barrier is reached by all eight.
constexpr int kClusterCtas = 8;
constexpr int kClThreads = 1024;
constexpr int kClBins = 256;
constexpr int kSubHists = 8;
constexpr int kMassSub = 4;            // copies of the mass histogram (64-bit bins)
constexpr int kMassBytes = (2 * kMassSub + 2 * kClusterCtas) * kClBins * 8;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of one of this CTA's shared variables in the CTA `rank` of the cluster
__device__ __forceinline__ uint32_t remote_addr(const void* p, uint32_t rank) {
    uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p)), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void remote_store(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void remote_store64(uint32_t addr, unsigned long long v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t remote_add(uint32_t addr, uint32_t v) {
    uint32_t old;
    asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
    return old;
}

__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kClThreads, 1)
sample_cluster_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ uniforms,
                      const int* __restrict__ recent, int recent_stride, const int* __restrict__ recent_len,
                      float temp, int top_k, float top_p, float rep_penalty, int* __restrict__ out, int per) {
    pdl_enter();      // the kernels before this one are complete from here on
    extern __shared__ float sl[];                              // this CTA's part of the row: `per` floats
    __shared__ float scratch[32];
    __shared__ float xf[2][kClusterCtas];                      // one float per CTA, two rounds in flight
    __shared__ uint32_t xhist[2][kClusterCtas][kClBins];       // every CTA's histogram, two passes in flight
    __shared__ uint32_t hist[kClBins];
    __shared__ uint32_t subhist[kSubHists][kClBins];
    __shared__ uint32_t xeq[kClusterCtas];
    __shared__ uint32_t sel[2];                                // chosen bin, what is still wanted
    __shared__ unsigned long long cand[kSmallSet];             // gathered in the first CTA
    __shared__ uint32_t n_cand;
    __shared__ uint32_t eq_here;
    const int tid = threadIdx.x;
    const int row = blockIdx.x / kClusterCtas;
    const uint32_t rank = cluster_rank();
    const int lo = (int)rank * per;
    const int n = max(0, min(per, V - lo));
    const float* l = logits + (size_t)row * ld + lo;

    if (tid == 0) { n_cand = 0; eq_here = 0; }
    if ((((size_t)row * ld + lo) & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        const int n4 = n >> 2;
        for (int i = tid; i < n4; i += kClThreads)
            reinterpret_cast<float4*>(sl)[i] = __ldg(reinterpret_cast<const float4*>(l) + i);
        for (int i = 4 * n4 + tid; i < n; i += kClThreads) sl[i] = l[i];
    } else {
        for (int i = tid; i < n; i += kClThreads) sl[i] = l[i];
    }
    __syncthreads();
    // repetition penalty, once per occurrence, on the copy
    if (tid == 0 && recent != nullptr && rep_penalty != 1.0f) {
        const int nrec = min(recent_len[row], 256);
        for (int j = 0; j < nrec; ++j) {
            const int t = recent[(size_t)row * recent_stride + j] - lo;
            if (t < 0 || t >= n) continue;
            const float v = sl[t];
            sl[t] = v > 0.f ? v / rep_penalty : v * rep_penalty;
        }
    }
    __syncthreads();

    int round = 0;
    // all CTAs' values of one float, in rank order, to every CTA
    auto share = [&](float mine, float (&all)[kClusterCtas]) {
        const int buf = round & 1;
        ++round;
        if (tid < kClusterCtas) remote_store(remote_addr(&xf[buf][rank], (uint32_t)tid), __float_as_uint(mine));
        cluster_sync_all();
#pragma unroll
        for (int r = 0; r < kClusterCtas; ++r) all[r] = xf[buf][r];
    };

    // ---- maximum and normaliser ----
    float m = -INFINITY;
    for (int i = tid; i < n; i += kClThreads) m = fmaxf(m, sl[i]);
    m = block_max(m, scratch);
    float all[kClusterCtas];
    share(m, all);
    float maxv = all[0];
#pragma unroll
    for (int r = 1; r < kClusterCtas; ++r) maxv = fmaxf(maxv, all[r]);
    float z = 0.f;
    for (int i = tid; i < n; i += kClThreads) z += expf((sl[i] - maxv) / temp);
    z = block_sum(z, scratch);
    share(z, all);
    z = 0.f;
#pragma unroll
    for (int r = 0; r < kClusterCtas; ++r) z += all[r];        // the same order in every CTA

    if (top_k <= 0 || top_k >= V) {
        // ---- no top_k: the whole row is kept (or its top_p prefix).  Probabilities are taken as integers,
        // p * 2^40, so that their sums do not depend on the order of addition: every CTA, every pass and
        // every run sees the same totals, and the radix selection by probability mass is exact in them.
        // per-CTA histograms are kept as three 32-bit sums of 14-bit limbs of the masses (a CTA holds fewer
        // than 2^17 tokens, so no limb sum overflows): 32-bit shared-memory atomics are native, 64-bit ones are not
        unsigned long long* msub = reinterpret_cast<unsigned long long*>(sl + per);            // [kMassSub][kClBins] (as 3 x u32 + pad)
        unsigned long long* xmass = msub + kMassSub * kClBins * 2;                              // [2][kClusterCtas][kClBins]
        uint32_t* limb = reinterpret_cast<uint32_t*>(msub);                                     // [kMassSub][kClBins][4]
        __shared__ unsigned long long xq[2][kClusterCtas];
        __shared__ unsigned long long msel[3];
        auto mass_of = [&](float logit) { return (unsigned long long)(expf((logit - maxv) / temp) * 1099511627776.0f); };
        int qround = 0;
        auto share_q = [&](unsigned long long mine, unsigned long long (&allq)[kClusterCtas]) {
            const int buf = qround & 1;
            ++qround;
            if (tid < kClusterCtas) remote_store64(remote_addr(&xq[buf][rank], (uint32_t)tid), mine);
            cluster_sync_all();
#pragma unroll
            for (int r = 0; r < kClusterCtas; ++r) allq[r] = xq[buf][r];
        };
        auto block_sum_q = [&](unsigned long long v) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            __syncthreads();
            if ((tid & 31) == 0) msub[tid >> 5] = v;
            __syncthreads();
            unsigned long long t = 0;
            for (int w = 0; w < kClThreads / 32; ++w) t += msub[w];
            __syncthreads();
            return t;
        };
        unsigned long long allq[kClusterCtas];
        unsigned long long zq = 0;
        for (int i = tid; i < n; i += kClThreads) zq += mass_of(sl[i]);
        share_q(block_sum_q(zq), allq);
        zq = 0;
#pragma unroll
        for (int r = 0; r < kClusterCtas; ++r) zq += allq[r];

        int pass_no = 0;
        // Selection by mass in the order "higher probability first, lower id first among equals":
        // strict: above <= target < above + mass(equals);  else: above < target <= above + mass(equals).
        // Returns the key, the mass above it and the number of tokens that have it.
        auto select = [&](unsigned long long target, bool strict, uint32_t& x, unsigned long long& above, uint32_t& n_equal) {
            uint32_t prefix = 0, mask = 0;
            above = 0;
            for (int pass = 0; pass < 4; ++pass, ++pass_no) {
                const int shift = 24 - 8 * pass, buf = pass_no & 1;
                for (int i = tid; i < kMassSub * kClBins * 4; i += kClThreads) limb[i] = 0;
                __syncthreads();
                uint32_t* mine = limb + (tid % kMassSub) * kClBins * 4;
                for (int i = tid; i < n; i += kClThreads) {
                    const float v = sl[i];
                    const uint32_t key = order_key(v);
                    if ((key & mask) == prefix) {
                        const unsigned long long q = mass_of(v);
                        uint32_t* bin = mine + ((key >> shift) & 255u) * 4;
                        atomicAdd(bin, (uint32_t)(q & 0x3FFFu));
                        atomicAdd(bin + 1, (uint32_t)((q >> 14) & 0x3FFFu));
                        atomicAdd(bin + 2, (uint32_t)(q >> 28));
                    }
                }
                __syncthreads();
                if (tid < kClBins) {
                    unsigned long long h = 0;
#pragma unroll
                    for (int c = 0; c < kMassSub; ++c) {
                        const uint32_t* bin = limb + (c * kClBins + tid) * 4;
                        h += (unsigned long long)bin[0] + ((unsigned long long)bin[1] << 14) + ((unsigned long long)bin[2] << 28);
                    }
#pragma unroll
                    for (uint32_t r = 0; r < kClusterCtas; ++r)
                        remote_store64(remote_addr(&xmass[(buf * kClusterCtas + rank) * kClBins + tid], r), h);
                }
                cluster_sync_all();
                if (tid < kClBins) {
                    unsigned long long t = 0;
#pragma unroll
                    for (int r = 0; r < kClusterCtas; ++r) t += xmass[(buf * kClusterCtas + r) * kClBins + tid];
                    msub[tid] = t;                         // the totals of this pass (the copies are spent)
                }
                __syncthreads();
                if (tid == 0) {
                    unsigned long long cum = above;
                    int b = kClBins - 1;
                    for (; b > 0; --b) {
                        const unsigned long long mb = msub[b];
                        if (strict ? (target < cum + mb) : (target <= cum + mb && mb > 0)) break;
                        cum += mb;
                    }
                    msel[0] = (unsigned long long)b;
                    msel[1] = cum;
                }
                __syncthreads();
                prefix |= (uint32_t)msel[0] << shift;
                mask |= 255u << shift;
                above = msel[1];
                __syncthreads();
            }
            x = prefix;
            // how many tokens have this key, over all CTAs (their masses are equal)
            uint32_t c = 0;
            for (int i = tid; i < n; i += kClThreads) c += (order_key(sl[i]) == x);
            unsigned long long allc[kClusterCtas];
            share_q(block_sum_q(c), allc);
            n_equal = 0;
#pragma unroll
            for (int r = 0; r < kClusterCtas; ++r) { n_equal += (uint32_t)allc[r]; xeq[r] = (uint32_t)allc[r]; }
        };

        uint32_t x = 0, n_equal = 0;
        unsigned long long above = 0;
        unsigned long long kept_mass = zq;
        if (top_p < 1.0f) {
            // the shortest prefix whose mass reaches top_p of the whole
            const unsigned long long target = (unsigned long long)((double)top_p * (double)zq);
            select(target > 0 ? target : 1, false, x, above, n_equal);
            const unsigned long long q_eq = mass_of(value_of_key(x));
            unsigned long long j = q_eq > 0 ? ((target > above ? target - above : 0) + q_eq - 1) / q_eq : 1;
            j = j < 1 ? 1 : (j > n_equal ? n_equal : j);
            kept_mass = above + j * q_eq;
        }
        const unsigned long long rr = (unsigned long long)((double)uniforms[row] * (double)kept_mass);
        select(rr < kept_mass ? rr : kept_mass - 1, true, x, above, n_equal);
        const unsigned long long q_eq = mass_of(value_of_key(x));
        unsigned long long j = q_eq > 0 ? (rr - above) / q_eq + 1 : 1;          // the j-th of the equals, by rising id
        j = j < 1 ? 1 : (j > n_equal ? n_equal : j);
        // which CTA holds the j-th equal, and which of its own it is
        uint32_t before = 0, owner = 0;
        for (uint32_t r = 0; r < kClusterCtas; ++r) {
            if (j <= before + xeq[r]) { owner = r; break; }
            before += xeq[r];
            owner = r;
        }
        if (rank == owner) {
            // this CTA's tokens with that key, collected (few as a rule), then the one with j' - 1 smaller ids among them
            int* ids = reinterpret_cast<int*>(msub);
            __shared__ uint32_t n_ids;
            const uint32_t mine_eq = xeq[rank], want_i = (uint32_t)(j - before);       // 1-based among this CTA's equals
            if (tid == 0) n_ids = 0;
            __syncthreads();
            if (mine_eq <= 2048) {
                for (int i = tid; i < n; i += kClThreads)
                    if (order_key(sl[i]) == x) ids[atomicAdd(&n_ids, 1u)] = lo + i;
                __syncthreads();
                for (uint32_t c = tid; c < mine_eq; c += kClThreads) {
                    const int id = ids[c];
                    uint32_t smaller = 0;
                    for (uint32_t d = 0; d < mine_eq; ++d) smaller += (ids[d] < id);
                    if (smaller == want_i - 1) out[row] = id;
                }
            } else if (tid == 0) {                              // a row of ties: walk it
                uint32_t seen = 0;
                for (int i = 0; i < n; ++i)
                    if (order_key(sl[i]) == x && ++seen == want_i) { out[row] = lo + i; break; }
            }
        }
        cluster_sync_all();
        return;
    }

    // ---- the top_k-th key by radix selection over all parts, 8 bits a pass ----
    uint32_t prefix = 0, mask = 0, want = (uint32_t)top_k;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass, buf = pass & 1;
        for (int i = tid; i < kSubHists * kClBins; i += kClThreads) (&subhist[0][0])[i] = 0;
        __syncthreads();
        // the leading bits of logits crowd into a few bins: several copies of the histogram, chosen
        // by the thread, keep the atomics from queueing up on one address
        uint32_t* mine = subhist[tid % kSubHists];
        for (int i = tid; i < n; i += kClThreads) {
            const uint32_t key = order_key(sl[i]);
            if ((key & mask) == prefix) atomicAdd(&mine[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid < kClBins) {
            uint32_t h = 0;
#pragma unroll
            for (int c = 0; c < kSubHists; ++c) h += subhist[c][tid];
#pragma unroll
            for (uint32_t r = 0; r < kClusterCtas; ++r) remote_store(remote_addr(&xhist[buf][rank][tid], r), h);
        }
        cluster_sync_all();
        if (tid < kClBins) {
            uint32_t t = 0;
#pragma unroll
            for (int r = 0; r < kClusterCtas; ++r) t += xhist[buf][r][tid];
            hist[tid] = t;
        }
        __syncthreads();
        if (tid < 32) {
            // one warp finds the bin, from the top: lane L holds bins 255-8L .. 248-8L
            uint32_t c[8], mine_sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * tid - j]; mine_sum += c[j]; }
            uint32_t incl = mine_sum;                       // counts of this lane's bins and of all higher bins
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
                if (tid >= o) incl += v;
            }
            uint32_t above = incl - mine_sum;
            const bool here = above < want && incl >= want;
            const bool last_resort = tid == 31 && incl < want;       // cannot happen while top_k <= the number of elements
            if (here || last_resort) {
                int j = 0;
                for (; j < 7; ++j) {
                    if (above + c[j] >= want) break;
                    above += c[j];
                }
                sel[0] = (uint32_t)(255 - 8 * tid - j);
                sel[1] = want - above;
            }
        }
        __syncthreads();
        prefix |= sel[0] << shift;
        mask |= 255u << shift;
        want = sel[1];
    }
    const uint32_t x = prefix;            // the top_k-th key; `want` of the tokens that have it are kept, lowest ids first

    // ---- how many of the equals each CTA holds ----
    {
        uint32_t c = 0;
        for (int i = tid; i < n; i += kClThreads) c += (order_key(sl[i]) == x);
        if (c) atomicAdd(&eq_here, c);
        __syncthreads();
        if (tid < kClusterCtas) remote_store(remote_addr(&xeq[rank], (uint32_t)tid), eq_here);
        cluster_sync_all();
    }
    uint32_t eq_before = 0;
    for (uint32_t r = 0; r < rank; ++r) eq_before += xeq[r];
    const uint32_t quota = eq_before >= want ? 0u : min(want - eq_before, xeq[rank]);   // equals this CTA contributes
    const bool all_equals = quota == xeq[rank];

    // ---- gather the kept tokens into the first CTA ----
    const uint32_t cand0 = remote_addr(&cand[0], 0), ncand0 = remote_addr(&n_cand, 0);
    auto push = [&](uint32_t key, int i) {
        const uint32_t at = remote_add(ncand0, 1u);
        if (at < (uint32_t)kSmallSet)
            remote_store64(cand0 + at * 8u, ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)(lo + i)));
    };
    for (int i = tid; i < n; i += kClThreads) {
        const uint32_t key = order_key(sl[i]);
        if (key > x || (key == x && all_equals)) push(key, i);
    }
    if (!all_equals && quota > 0 && tid == 0) {          // a tie across the cut inside this part: the lowest ids, in order
        uint32_t taken = 0;
        for (int i = 0; i < n && taken < quota; ++i)
            if (order_key(sl[i]) == x) { push(x, i); ++taken; }
    }
    cluster_sync_all();
    if (rank != 0) return;

    // ---- the first CTA: sort and walk ----
    const int nk = min((int)n_cand, kSmallSet);
    int n2 = 1;
    while (n2 < nk) n2 <<= 1;
    for (int i = nk + tid; i < n2; i += kClThreads) cand[i] = 0ull;        // padding sorts last
    __syncthreads();
    for (int k = 2; k <= n2; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < n2; i += kClThreads) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = cand[i], b = cand[ixj];
                    const bool desc = (i & k) == 0;
                    if (desc ? (a < b) : (a > b)) { cand[i] = b; cand[ixj] = a; }
                }
            }
            __syncthreads();
        }
    if (tid == 0) {
        auto prob_of = [&](unsigned long long c) { return expf((value_of_key((uint32_t)(c >> 32)) - maxv) / temp) / z; };
        int cut = nk;
        if (top_p < 1.0f) {
            float cum = 0.f;
            for (int i = 0; i < nk; ++i) {
                cum += prob_of(cand[i]);
                if (cum >= top_p) { cut = i + 1; break; }
            }
        }
        float total = 0.f;
        for (int i = 0; i < cut; ++i) total += prob_of(cand[i]);
        const float rr = uniforms[row] * total;
        float cdf = 0.f;
        int pick = cut - 1;
        for (int i = 0; i < cut; ++i) {
            cdf += prob_of(cand[i]);
            if (rr < cdf) { pick = i; break; }
        }
        out[row] = (int)(~(uint32_t)(cand[pick] & 0xffffffffull));
    }
}

// Arg max alone (first maximum wins), for the greedy loop: reads, never writes, the logits.
// A row is cut into chunks, one block each; a block leaves its (maximum, id) in `partial`
// and takes a ticket; the block that takes a row's last ticket reduces the row's partials
// and puts the counter back to zero for the next launch.
constexpr int kArgmaxThreads = 256;

__device__ __forceinline__ void argmax_merge(float& best, int& best_i, float ov, int oi) {
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
}

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int chunk, float* __restrict__ partial_val,
              int* __restrict__ partial_idx, int* __restrict__ tickets, int* __restrict__ out,
              const int* __restrict__ recent, int recent_stride, const int* __restrict__ recent_len, float rep_penalty) {
    pdl_enter();      // the kernels before this one are complete from here on
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ int si[kArgmaxThreads / 32];
    __shared__ int is_last;
    __shared__ int pen_id[256];          // recent tokens that lie in this chunk, each once,
    __shared__ float pen_val[256];       // with their logits after the penalty (once per occurrence)
    __shared__ int n_pen;
    const int row = blockIdx.y, nchunks = gridDim.x;
    const float* l = logits + (size_t)row * ld;
    const int lo = blockIdx.x * chunk, hi = min(V, lo + chunk);
    // The penalty is applied once per occurrence; a logit keeps its sign under it, so the order of the
    // occurrences does not matter and each distinct token is handled by the thread of its first occurrence.
    __shared__ int rec[256];
    const int nrec = (recent != nullptr && rep_penalty != 1.0f) ? min(recent_len[row], 256) : 0;
    if (threadIdx.x == 0) n_pen = 0;
    if ((int)threadIdx.x < nrec) rec[threadIdx.x] = recent[(size_t)row * recent_stride + threadIdx.x];
    __syncthreads();
    if ((int)threadIdx.x < nrec) {
        const int t = rec[threadIdx.x];
        if (t >= lo && t < hi) {
            int times = 0;
            bool first = true;
            for (int j = 0; j < nrec; ++j) {
                if (rec[j] != t) continue;
                if (j < (int)threadIdx.x) first = false;
                ++times;
            }
            if (first) {
                float v = l[t];
                for (int k = 0; k < times; ++k) v = v > 0.f ? v / rep_penalty : v * rep_penalty;
                const int at = atomicAdd(&n_pen, 1);
                pen_id[at] = t;
                pen_val[at] = v;
            }
        }
    }
    __syncthreads();
    const int np = n_pen;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += kArgmaxThreads) {
        float v = l[i];
        for (int e = 0; e < np; ++e)
            if (pen_id[e] == i) v = pen_val[e];
        if (v > best) { best = v; best_i = i; }     // ids rise within a thread: first maximum kept
    }
    auto block_reduce = [&]() {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            argmax_merge(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
        if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
        __syncthreads();
        if (threadIdx.x < 32) {
            best = threadIdx.x < kArgmaxThreads / 32 ? sv[threadIdx.x] : -INFINITY;
            best_i = threadIdx.x < kArgmaxThreads / 32 ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                argmax_merge(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
        }
    };
    block_reduce();
    if (threadIdx.x == 0) {
        partial_val[(size_t)row * nchunks + blockIdx.x] = best;
        partial_idx[(size_t)row * nchunks + blockIdx.x] = best_i;
        __threadfence();
        is_last = atomicAdd(&tickets[row], 1) == nchunks - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    best = -INFINITY;
    best_i = 0x7fffffff;
    for (int c = threadIdx.x; c < nchunks; c += kArgmaxThreads)
        argmax_merge(best, best_i, __ldcg(&partial_val[(size_t)row * nchunks + c]), __ldcg(&partial_idx[(size_t)row * nchunks + c]));
    __syncthreads();
    block_reduce();
    if (threadIdx.x == 0) {
        out[row] = best_i == 0x7fffffff ? 0 : best_i;
        tickets[row] = 0;
    }
}

// Tests switch the cluster kernel off to put the one-CTA kernel through the same cases.
static int g_cluster_sampler = 1;
static bool cluster_sampler_enabled() { return g_cluster_sampler != 0; }

}  // namespace hos

using namespace hos;

extern "C" void hos_sample_use_cluster(int on) { g_cluster_sampler = on ? 1 : 0; }

// Chunks a row is cut into, and the floats of workspace the arg max needs: partial maxima
// and ids, [B][chunks] each.  `tickets` is B ints that are zero before the first launch.
extern "C" int hos_argmax_chunks(int V) {
    int c = (V + 4095) / 4096;
    return c < 1 ? 1 : (c > 256 ? 256 : c);
}
// recent, recent_len, rep_penalty: the repetition penalty of the sampler (once per occurrence of a recent
// token), applied on the fly; recent == NULL or rep_penalty == 1: none.  The logits are not written.
extern "C" int hos_argmax(const float* logits, int ld, int B, int V, int* out, float* workspace, int* tickets,
                          const int* recent, int recent_stride, const int* recent_len, float rep_penalty,
                          cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) HOS_REFUSE("argmax: empty vocabulary");
    if (B > 65535) HOS_REFUSE("argmax: %d rows are more than one launch takes", B);
    if (!(rep_penalty > 0.f)) HOS_REFUSE("argmax: repetition penalty must be positive");
    const int chunks = hos_argmax_chunks(V);
    const int chunk = (V + chunks - 1) / chunks;
    dim3 grid(chunks, B);
    launch_pdl(argmax_kernel, dim3(grid), dim3(kArgmaxThreads), 0, stream, logits, ld, V, chunk, workspace,
                                                      reinterpret_cast<int*>(workspace + (size_t)B * chunks), tickets, out,
                                                      recent, recent_stride, recent_len, rep_penalty);
    return check_launch("argmax");
}

// recent: [B, recent_stride] token ids with recent_len[b] valid entries per row (may be NULL).
extern "C" int hos_sample(float* logits, int ld, int B, int V, const float* uniforms,
                          const int* recent, int recent_stride, const int* recent_len, float temp,
                          int top_k, float top_p, float rep_penalty, int* out, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) HOS_REFUSE("sample: empty vocabulary");
    if (V > (1 << 24)) HOS_REFUSE("sample: vocabulary %d is beyond 2^24 (counts are kept in float)", V);
    if (top_k < 0) HOS_REFUSE("sample: top_k %d is negative", top_k);
    if (!(rep_penalty > 0.f)) HOS_REFUSE("sample: repetition penalty must be positive");
    // temperature sampling (from the top_k most probable, up to 1024 of them, or from the whole row or its
    // top_p prefix): a cluster of CTAs per row, each with its part of the row in shared memory
    {
        const int per = ((V + kClusterCtas - 1) / kClusterCtas + 3) / 4 * 4;
        size_t need = (size_t)per * sizeof(float);
        const bool no_top_k = top_k <= 0 || top_k >= V;
        if (no_top_k) need += kMassBytes;
        if (temp > 0.f && (no_top_k || top_k <= kSmallSet) && need <= 190 * 1024 && cluster_sampler_enabled()) {
            static size_t attr_cluster = 0;
            if (need > attr_cluster) {
                if (cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need) != cudaSuccess)
                    HOS_REFUSE("sample: cannot get %zu bytes of shared memory", need);
                attr_cluster = need;
            }
            launch_pdl(sample_cluster_kernel, dim3(B * kClusterCtas), dim3(kClThreads), need, stream, (const float*)logits, ld, V,
                       uniforms, recent, recent_stride, recent_len, temp, top_k, top_p, rep_penalty, out, per);
            return check_launch("sample");
        }
    }
    const size_t smem = (size_t)(kBins * kThreads + kBins + 32) * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
    }
    launch_pdl(sample_kernel, dim3(B), dim3(kThreads), smem, stream, logits, ld, V, uniforms, recent, recent_stride,
                                                 recent_len, temp, top_k, top_p, rep_penalty, out);
    return check_launch("sample");
}
