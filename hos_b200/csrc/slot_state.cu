// The per-slot record: what a sequence keeps on the device besides keys and values.
//
// Every slot of the cache has kSlotWords 32-bit words,
//   [0] pos        tokens the sequence holds (its next token's position)
//   [1] last       the token sampled last (the next step's input)
//   [2] flags      bit 0: finished (sampled a stop token, or has all the tokens it may have)
//   [3] count      tokens sampled so far
//   [4],[5]        state of the sequence's xorshift64 generator (low, high word)
//   [6] limit      most tokens to sample (0: no limit)
//   [7]            spare
// and a ring of the kRecentMax tokens sampled last (what the repetition penalty looks at).
// The reference keeps the same things on the host: the position beside the cache
// (src/forward.rs:146-162, src/lib.rs:175-184) and the generator and the recent tokens as
// locals of its generation loop (src/lib.rs:404-448).  Here a decode step reads its input
// token and its position from the record and writes the sampled token back, so that a
// generation loop never waits for the host between steps.
#include "common.cuh"

namespace hos {

constexpr int kSlotWords = 8;
constexpr int kRecentMax = 256;
enum { kPos = 0, kLast = 1, kFlags = 2, kCount = 3, kRngLo = 4, kRngHi = 5, kLimit = 6 };
// what slot_begin does
constexpr int kBeginAdvance = 1;          // hand out the position and move it on by one
constexpr int kBeginTokenFromRecord = 2;  // the step's input token is the record's last token (else: the caller's)
constexpr int kBeginUniform = 4;          // draw the next number of the sequence's generator
constexpr int kBeginRecent = 8;           // hand out the last tokens for the repetition penalty
constexpr int kBeginSkipFinished = 16;    // a finished sequence's row becomes padding

// meta: [0] live rows, [1] number of stop ids, [2..2+kMaxStops) stop ids
constexpr int kMaxStops = 16;

// One warp per row of a single-token step of up to B rows; row b belongs to slot slots[b].
__global__ void slot_begin_kernel(int* __restrict__ record, const int* __restrict__ ring,
                                  const int* __restrict__ slots, const int* __restrict__ meta, int B, int flags,
                                  int* __restrict__ tokens, int* __restrict__ pos, int* __restrict__ after,
                                  int* __restrict__ seq, int* __restrict__ cu, float* __restrict__ uniforms,
                                  int* __restrict__ recent, int* __restrict__ recent_len, int n_recent) {
    pdl_enter();
    const int b = blockIdx.x, lane = threadIdx.x;
    const int live = min(meta[0], B);
    if (lane == 0) {
        cu[b] = min(b, live);
        if (b == B - 1) cu[B] = live;
    }
    if (b >= live) {                       // padding row
        if (lane == 0) {
            tokens[b] = -1; pos[b] = 0; after[b] = 1; seq[b] = -1;
            if (uniforms) uniforms[b] = 0.f;
            if (recent_len) recent_len[b] = 0;
        }
        return;
    }
    const int slot = slots[b];
    int* r = record + (size_t)slot * kSlotWords;
    const bool finished = (r[kFlags] & 1) != 0;
    const int count = r[kCount];
    if ((flags & kBeginRecent) && recent != nullptr) {
        const int len = min(min(count, n_recent), kRecentMax);
        for (int i = lane; i < n_recent; i += 32)
            recent[(size_t)b * n_recent + i] =
                i < len ? ring[(size_t)slot * kRecentMax + ((count - len + i) % kRecentMax)] : -1;
        if (lane == 0) recent_len[b] = len;
    }
    if (lane != 0) return;
    const bool skip = finished && (flags & kBeginSkipFinished);
    if (flags & kBeginAdvance) {
        const int p = r[kPos];
        pos[b] = p;
        after[b] = p + 1;
        if (!skip) r[kPos] = p + 1;
        if (flags & kBeginTokenFromRecord) tokens[b] = r[kLast];
        seq[b] = skip ? -1 : b;
    }
    if ((flags & kBeginUniform) && uniforms != nullptr) {
        // xorshift64 (13, 7, 17); the top 24 bits give a number in [0, 1)  (src/lib.rs:78-85)
        unsigned long long x = ((unsigned long long)(unsigned)r[kRngHi] << 32) | (unsigned)r[kRngLo];
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        if (!finished) {
            r[kRngLo] = (int)(unsigned)(x & 0xffffffffull);
            r[kRngHi] = (int)(unsigned)(x >> 32);
        }
        uniforms[b] = (float)(x >> 40) / 16777216.0f;
    }
}

// After sampling: the token becomes the record's last token and joins the recent ones; a stop
// token, or the last token the sequence may have, marks it finished.
__global__ void slot_end_kernel(int* __restrict__ record, int* __restrict__ ring, const int* __restrict__ slots,
                                const int* __restrict__ meta, int B, const int* __restrict__ sampled) {
    pdl_enter();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= min(meta[0], B)) return;
    const int slot = slots[b];
    int* r = record + (size_t)slot * kSlotWords;
    if (r[kFlags] & 1) return;
    const int t = sampled[b], count = r[kCount];
    r[kLast] = t;
    ring[(size_t)slot * kRecentMax + (count % kRecentMax)] = t;
    r[kCount] = count + 1;
    bool stop = r[kLimit] > 0 && count + 1 >= r[kLimit];
    const int n_stop = min(meta[1], kMaxStops);
    for (int i = 0; i < n_stop; ++i) stop = stop || meta[2 + i] == t;
    if (stop) r[kFlags] |= 1;
}

// The sequences of a step of many tokens now hold seq_len_after tokens (sequences that brought none
// are left alone).
__global__ void slot_set_pos_kernel(int* __restrict__ record, const int* __restrict__ seq_slot,
                                    const int* __restrict__ seq_len_after, const int* __restrict__ cu_seqlens,
                                    int n_seqs) {
    pdl_enter();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seqs || cu_seqlens[s + 1] <= cu_seqlens[s]) return;
    record[(size_t)seq_slot[s] * kSlotWords + kPos] = seq_len_after[s];
}

// Whole records written from values[n][kSlotWords]: the words whose bit is set in word_mask.
__global__ void slot_write_kernel(int* __restrict__ record, const int* __restrict__ slots,
                                  const int* __restrict__ values, int word_mask, int n) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * kSlotWords) return;
    const int w = i % kSlotWords;
    if (word_mask >> w & 1) record[(size_t)slots[i / kSlotWords] * kSlotWords + w] = values[i];
}

}  // namespace hos

using namespace hos;

extern "C" int hos_slot_words() { return kSlotWords; }
extern "C" int hos_slot_recent_max() { return kRecentMax; }
extern "C" int hos_slot_max_stops() { return kMaxStops; }

extern "C" int hos_slot_begin(int* record, const int* ring, const int* slots, const int* meta, int B, int flags,
                              int* tokens, int* pos, int* after, int* seq, int* cu, float* uniforms, int* recent,
                              int* recent_len, int n_recent, cudaStream_t stream) {
    if (B <= 0) return 0;
    if ((flags & kBeginRecent) && (n_recent < 1 || n_recent > kRecentMax))
        HOS_REFUSE("slot_begin: %d recent tokens asked for, the record keeps %d", n_recent, kRecentMax);
    launch_pdl(slot_begin_kernel, dim3(B), dim3(32), 0, stream, record, ring, slots, meta, B, flags, tokens, pos, after,
               seq, cu, uniforms, recent, recent_len, n_recent);
    return check_launch("slot_begin");
}

extern "C" int hos_slot_end(int* record, int* ring, const int* slots, const int* meta, int B, const int* sampled,
                            cudaStream_t stream) {
    if (B <= 0) return 0;
    launch_pdl(slot_end_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, record, ring, slots, meta, B, sampled);
    return check_launch("slot_end");
}

extern "C" int hos_slot_set_pos(int* record, const int* seq_slot, const int* seq_len_after, const int* cu_seqlens,
                                int n_seqs, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    launch_pdl(slot_set_pos_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, stream, record, seq_slot, seq_len_after,
               cu_seqlens, n_seqs);
    return check_launch("slot_set_pos");
}

extern "C" int hos_slot_write(int* record, const int* slots, const int* values, int word_mask, int n,
                              cudaStream_t stream) {
    if (n <= 0) return 0;
    launch_pdl(slot_write_kernel, dim3((n * kSlotWords + 127) / 128), dim3(128), 0, stream, record, slots, values,
               word_mask, n);
    return check_launch("slot_write");
}
