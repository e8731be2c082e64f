// Token selection for one row by a team of THREADS threads (a whole CTA, or the worker warps of the
// persistent tick kernel). Vocabulary at most 4096.
//
// The chain is the one of crates/omni-qwen3-tts/kernels/talker.cu:108-293: repetition penalty and
// suppression on the raw logits, temperature, top-k with ties kept (the k-th largest found by a radix
// select over order-preserving integer keys), softmax numerators with __expf, and an inverse-CDF walk
// in vocabulary order against one uniform. The reference runs 1024 threads with four consecutive
// logits each, and the association order of its block scan decides which token a uniform lands on.
// That order is reproduced here for any team size by scanning 1024 *virtual* threads: per-virtual-
// thread sum of four, a Hillis-Steele inclusive scan over each group of 32 virtual lanes, the same
// scan over the 32 group totals, exclusive prefix formed as (group_before + inclusive) - own.
// Not in the reference: top_p < 1 (nucleus filter after top-k) and uniforms from Philox4x32-10.
#pragma once
#include "util.cuh"

namespace omni {
namespace sampler {

constexpr int kVocabMax = 4096;
constexpr int kVirtualThreads = 1024;  // the reference's block size
constexpr int kVirtualPer = 4;         // logits per virtual thread
constexpr int kMaxNucleus = 1024;

struct CtaSync {
  static __device__ __forceinline__ void sync() { __syncthreads(); }
};

template <int ID, int COUNT>
struct NamedSync {
  static __device__ __forceinline__ void sync() { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory"); }
};

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Philox4x32-10, counter (frame, group, 0, 0), key = the sequence's seed; first word -> [0, 1) with 24 bits.
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t frame, uint32_t group) {
  uint32_t c0 = frame, c1 = group, c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
    const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
    c0 = n0, c1 = l1, c2 = n2, c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

struct Shared {
  alignas(16) uint32_t hist[4][256];  // one set of digit counters per pass of the k-th key selection
  uint32_t warp_cnt[32];
  float red[32];
  float wtot[32];
  float vscan[kVirtualThreads];
  int token, last;
  unsigned long long best;
  int n_cand;
  alignas(16) int cand_idx[kMaxNucleus];  // 16-byte aligned: the four arrays from here on also stage a row of logits
  float cand_p[kMaxNucleus];
  int sorted_idx[kMaxNucleus];
  float sorted_p[kMaxNucleus];
  uint32_t drop[kVocabMax / 32];
};

struct Params {
  int vocab;
  float temperature;
  int top_k;
  float top_p;
  float penalty;
  int suppress_lo, suppress_hi, exempt, min_frames;
  int penalize;
  int group;
  int philox;
  int seen_words;
};

// Team thread `tid` owns the PER = 4096 / THREADS consecutive logits starting at tid * PER.
template <int THREADS, typename Sync>
struct Team {
  static constexpr int PER = kVocabMax / THREADS;
  static constexpr int VPT = kVirtualThreads / THREADS;  // virtual threads per team thread
  static_assert(PER % kVirtualPer == 0 && THREADS >= 128 && THREADS <= kVirtualThreads, "team size");
  static_assert(32 % PER == 0, "a thread's logits share one word of the seen bitmap");

  // The word of the sequence's seen bitmap that covers this thread's logits (0 when nothing is penalised).
  static __device__ __forceinline__ uint32_t seen_word(const int32_t* slot, const Params& prm, int tid) {
    const uint32_t* seen = reinterpret_cast<const uint32_t*>(slot + 16);
    return prm.penalize && tid * PER < prm.vocab ? seen[tid * PER / 32] : 0u;
  }

  static __device__ float team_max(float v, int tid, Shared& sh) {
    v = warp_fmax(v);
    if ((tid & 31) == 0) sh.red[tid >> 5] = v;
    Sync::sync();
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) m = fmaxf(m, sh.red[w]);
    Sync::sync();
    return m;
  }

  // The k-th largest key of the row (ties share it), most significant digit first, eight bits at a time. Logits are
  // a few units wide, so the keys' leading digits take a handful of values: counted one atomic per key, that pass would
  // serialise thousands of additions on two or three shared-memory words, so the first digit is found by counting
  // (below). The other passes count through shared-memory atomics; every pass has its own 256 counters (zeroed once,
  // up front), and after the pass's one team barrier EVERY warp picks the digit by itself from the counters (lane l
  // sums counters 8l .. 8l + 7, a shuffle scan gives the keys above each lane's range).
  static __device__ uint32_t kth_largest_key(const uint32_t* key, int vocab, uint32_t k, uint32_t top_digit, int tid,
                                             Shared& sh) {
    uint32_t prefix = 0, left = k;
    const int lane = tid & 31;
    for (int i = tid; i < 4 * 256; i += THREADS) (&sh.hist[0][0])[i] = 0;
    // First digit: the keys' leading bytes take two or three values just below the largest key's (`top_digit`), so
    // they are not counted through shared-memory atomics at all: from the top byte downwards, every thread counts
    // its own keys with that byte and the team adds the counts, until the k-th key's byte is reached.
    for (uint32_t d = top_digit;; --d) {
      uint32_t mine = 0;
#pragma unroll
      for (int j = 0; j < PER; ++j) mine += tid * PER + j < vocab && key[j] >> 24 == d ? 1u : 0u;
      mine = __reduce_add_sync(0xffffffffu, mine);
      Sync::sync();  // (also orders the zeroing above, and the previous round's reads, before the writes below)
      if (lane == 0) sh.warp_cnt[tid >> 5] = mine;
      Sync::sync();
      uint32_t total = 0;
#pragma unroll
      for (int w = 0; w < THREADS / 32; ++w) total += sh.warp_cnt[w];
      if (total >= left || d == 0) {
        prefix = d << 24;
        break;
      }
      left -= total;
    }
    for (int pass = 1; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      uint32_t* hist = sh.hist[pass];
      const uint32_t fixed = 0xffffffffu << (shift + 8);
      // only the keys that carry the digits fixed so far count, spread over the counters
#pragma unroll
      for (int j = 0; j < PER; ++j)
        if (tid * PER + j < vocab && ((key[j] ^ prefix) & fixed) == 0) atomicAdd(&hist[(key[j] >> shift) & 255u], 1u);
      Sync::sync();
      // at_least[d] = keys whose digit is >= d; the digit wanted is the one with at_least - count < left <= at_least
      uint32_t c[8];
      *reinterpret_cast<uint4*>(&c[0]) = *reinterpret_cast<const uint4*>(&hist[8 * lane]);
      *reinterpret_cast<uint4*>(&c[4]) = *reinterpret_cast<const uint4*>(&hist[8 * lane + 4]);
      uint32_t mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine += c[j];
      uint32_t incl = mine;  // keys in this lane's counters and in those of the lanes above it
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t other = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += other;
      }
      uint32_t at_least = incl - mine, digit = 0, new_left = 0;
      bool found = false;
#pragma unroll
      for (int j = 7; j >= 0; --j) {
        const uint32_t above = at_least;
        at_least += c[j];
        if (!found && above < left && at_least >= left) {
          found = true;
          digit = 8u * lane + j;
          new_left = left - above;
        }
      }
      const uint32_t who = __ballot_sync(0xffffffffu, found);  // exactly one lane
      const int src = __ffs(who) - 1;
      prefix |= __shfl_sync(0xffffffffu, digit, src) << shift;
      left = __shfl_sync(0xffffffffu, new_left, src);
    }
    return prefix;
  }

  // v: this thread's PER processed logits (-inf beyond the vocabulary).
  static __device__ int draw(const float* v, int vocab, float temperature, int top_k, float top_p, float u, int tid,
                             Shared& sh) {
    if (temperature <= 0.f) {  // argmax, lowest index on ties (talker.cu:177-188)
      if (tid == 0) sh.best = 0ull;
      Sync::sync();
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid * PER + j;
        if (i < vocab) atomicMax(&sh.best, (unsigned long long)order_key(v[j]) << 32 | (uint32_t)(4095 - i));
      }
      Sync::sync();
      const int token = 4095 - (int)(sh.best & 0xffffffffull);
      Sync::sync();
      return token;
    }
    float x[PER];
    uint32_t key[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      x[j] = v[j] / temperature;
      key[j] = order_key(x[j]);
      mx = fmaxf(mx, x[j]);
    }
    const int keep = top_k > 0 && top_k < vocab ? top_k : vocab;
    const float m = team_max(mx, tid, sh);
    const uint32_t threshold = keep < vocab ? kth_largest_key(key, vocab, (uint32_t)keep, order_key(m) >> 24, tid, sh) : 0u;
    float p[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) p[j] = tid * PER + j < vocab && key[j] >= threshold ? __expf(x[j] - m) : 0.f;

    if (top_p < 1.f) {
      // compact the survivors, rank them by (probability desc, index asc), walk the ranking once
      // and drop every token whose preceding mass already reaches top_p
      if (tid == 0) sh.n_cand = 0;
      for (int i = tid; i < kVocabMax / 32; i += THREADS) sh.drop[i] = 0u;
      Sync::sync();
#pragma unroll
      for (int j = 0; j < PER; ++j)
        if (p[j] > 0.f) {
          const int at = atomicAdd(&sh.n_cand, 1);
          if (at < kMaxNucleus) {
            sh.cand_idx[at] = tid * PER + j;
            sh.cand_p[at] = p[j];
          }
        }
      Sync::sync();
      const int nc = min(sh.n_cand, kMaxNucleus);
      for (int a = tid; a < nc; a += THREADS) {
        const float pa = sh.cand_p[a];
        const int ia = sh.cand_idx[a];
        int rank = 0;
        for (int b = 0; b < nc; ++b) {
          const float pb = sh.cand_p[b];
          rank += (pb > pa) || (pb == pa && sh.cand_idx[b] < ia);
        }
        sh.sorted_idx[rank] = ia;
        sh.sorted_p[rank] = pa;
      }
      Sync::sync();
      if (tid == 0) {
        float tot = 0.f;
        for (int r = 0; r < nc; ++r) tot += sh.sorted_p[r];
        float before = 0.f;
        for (int r = 0; r < nc; ++r) {
          const float mine = sh.sorted_p[r];
          if (r > 0 && before >= top_p * tot) {
            const int idx = sh.sorted_idx[r];
            sh.drop[idx >> 5] |= 1u << (idx & 31);
          }
          before += mine;
        }
      }
      Sync::sync();
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid * PER + j;
        if (sh.drop[i >> 5] >> (i & 31) & 1u) p[j] = 0.f;
      }
    }

    // --- the reference's block scan over 1024 virtual threads (talker.cu:136-169) ---
    // A virtual warp is 32 / VPT neighbouring lanes of a real warp, each holding VPT consecutive virtual lanes, so the
    // reference's shuffle scan (x[i] += x[i - o] for o = 1, 2, 4, 8, 16, every lane reading the values of the step
    // before) runs on real shuffles: a source o < VPT lanes back sits in this thread or in the lane before it, a
    // source o >= VPT lanes back o / VPT lanes before, in the same slot. Same additions in the same order.
    float own[VPT], incl[VPT];
#pragma unroll
    for (int q = 0; q < VPT; ++q) {
      float o = 0.f;
#pragma unroll
      for (int e = 0; e < kVirtualPer; ++e) o += p[q * kVirtualPer + e];
      own[q] = incl[q] = o;
    }
    if (tid == 0) {
      sh.token = -1;
      sh.last = 0;
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float up[VPT];
#pragma unroll
      for (int q = 0; q < VPT; ++q) {
        if (o >= VPT) {
          up[q] = __shfl_up_sync(0xffffffffu, incl[q], o / VPT);
        } else {
          const float before = __shfl_up_sync(0xffffffffu, incl[(q + VPT - o) % VPT], 1);
          up[q] = q >= o ? incl[q - o] : before;
        }
      }
#pragma unroll
      for (int q = 0; q < VPT; ++q)
        if (((tid * VPT + q) & 31) >= o) incl[q] += up[q];
    }
    if (((tid * VPT + VPT - 1) & 31) == 31) sh.vscan[tid * VPT + VPT - 1] = incl[VPT - 1];  // a virtual warp's total
    Sync::sync();
    if (tid < 32) {  // the same scan over the 32 group totals
      float wsum = sh.vscan[tid * 32 + 31];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, wsum, o);
        if (tid >= o) wsum += up;
      }
      sh.wtot[tid] = wsum;
    }
    Sync::sync();
    const float total = sh.wtot[31];
    const float target = u * total;
#pragma unroll
    for (int q = 0; q < VPT; ++q) {
      const int vt = tid * VPT + q, vw = vt >> 5;
      const float before = vw > 0 ? sh.wtot[vw - 1] : 0.f;
      float run = before + incl[q] - own[q];
#pragma unroll
      for (int e = 0; e < kVirtualPer; ++e) {
        const float pe = p[q * kVirtualPer + e];
        const int i = vt * kVirtualPer + e;
        if (pe > 0.f) {
          atomicMax(&sh.last, i);
          if (run <= target && target < run + pe) atomicMax(&sh.token, i);
        }
        run += pe;
      }
    }
    Sync::sync();
    const int token = sh.token >= 0 ? sh.token : sh.last;
    Sync::sync();
    return token;
  }

  // `talker_sample` (talker.cu:259-293) for one row. `load(i, j)` returns logit i = tid * PER + j as f32 (already rounded
  // to bf16 by the caller). slot: i32 last_frame[16] | u32 seen[seen_words] | u64 seed (8-byte aligned).
  // `seen_bits` = seen_word() of this thread, read before the call (so callers can fetch it early).
  // Returns the token (identical in every team thread); thread 0 writes codes, the slot and the bitmap.
  template <typename Load>
  static __device__ int sample_row(Load load, const Params& prm, int frame, float uniform, int forced, int32_t* slot,
                                   uint32_t seen_bits, int32_t* code_out, int tid, Shared& sh) {
    uint32_t* seen = reinterpret_cast<uint32_t*>(slot + 16);
    int token = forced;
    if (forced < 0) {
      const bool exempt_blocked = frame < prm.min_frames;
      float v[PER];
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = tid * PER + j;
        float x = -INFINITY;
        if (i < prm.vocab) {
          x = load(i, j);
          if (seen_bits >> (i % 32) & 1u) x = x > 0.f ? x / prm.penalty : x * prm.penalty;
          const bool in_range = i >= prm.suppress_lo && i < prm.suppress_hi;
          if ((in_range && i != prm.exempt) || (i == prm.exempt && exempt_blocked)) x = -INFINITY;
        }
        v[j] = x;
      }
      float u = uniform;
      if (prm.philox) {
        const uint64_t seed = *reinterpret_cast<const uint64_t*>(seen + prm.seen_words + (prm.seen_words & 1));
        u = philox_uniform(seed, (uint32_t)frame, (uint32_t)prm.group);
      }
      token = min(max(draw(v, prm.vocab, prm.temperature, prm.top_k, prm.top_p, u, tid, sh), 0), prm.vocab - 1);
    }
    Sync::sync();  // every thread has read the bitmap before it changes
    if (tid == 0) {
      *code_out = token;
      slot[prm.group] = token;
      if (prm.penalize) seen[token / 32] |= 1u << (token % 32);
    }
    return token;
  }
};

}  // namespace sampler
}  // namespace omni
