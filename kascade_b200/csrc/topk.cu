// Exact per-row Top-k (one CTA per row): the k-th largest score is bracketed from a sample, the few
// candidates inside the bracket are selected among exactly in shared memory, and the selected positions are
// written in ascending index order.
//
// Replaces the torch.topk call sites of the reference's efficient path
// (strategies/EfficientKascadeStrategy.py:82,90,111).
//
//   1. Bracket: 4096 (8192 for rows beyond 65536) evenly spaced samples of the row go into a 512-bin histogram
//      over the samples' own key range, and those in the bins around the sample ranks k/n * samples -/+
//      (5 sigma + 16) into a second one over just these bins; its bins give two keys lo <= hi.
//   2. One pass over the row: every warp owns a contiguous piece of it, counts its scores above hi and appends
//      its keys in [lo, hi] (a few per cent of the row) to a list of its own in shared memory.  If
//      count(> hi) < k <= count(> hi) + |lists|  and the lists fit, the k-th largest score is the
//      (k - count(> hi))-th largest of the lists: a radix select over them (9-bit digits of key - lo, only as
//      many as hi - lo has bits) finds it exactly, and every warp learns from its own list how many of its scores
//      lie above / at the threshold.  Rows of up to 4096 scores skip the sample: the whole row goes to the lists.
//   3. Otherwise (the sample misjudged the row, which the check above detects, or a list overflowed) the k-th
//      largest key is found by four 9/9/9/5-bit histogram passes over the row itself, and a counting pass
//      gives the warps their numbers.
//   4. The last pass writes the selected positions of every warp's piece in index order, with warp-local prefix
//      sums only, taking ties at the threshold from the lowest index upwards.
// The row is read from HBM once; the later passes find it in L1 / L2.
#include "common.cuh"

namespace kb200 {

constexpr int kTopkThreads = 512;
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kDigit = 9;
constexpr int kTopkBins = 1 << kDigit;                            // 9-bit digits: one warp can search a histogram
constexpr int kCandCap = 8192;                            // keys the candidate lists hold, one list per warp
constexpr int kWarpList = kCandCap / kTopkWarps;          // 512
constexpr int kListRow = 4096;                            // rows up to this length are selected from directly
constexpr int kTopkUnroll = 4;                            // 16-byte loads a lane keeps in flight in the streaming passes

// order-preserving map float -> uint32 (larger float <=> larger key)
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);   // flips all bits of a negative, the sign of the rest
}
// Keys of one 16-byte piece.  Positions beyond the row (only the row's last piece has any, and the lanes past
// the end) get key 0, which no score has (it would be a NaN with all bits set) and which the passes below never
// count: they compare against keys >= 1.
__device__ __forceinline__ void piece_keys(const float4& x, int i4, int n4, int n, uint32_t (&u)[4]) {
  u[0] = float_key(x.x); u[1] = float_key(x.y); u[2] = float_key(x.z); u[3] = float_key(x.w);
  if (i4 >= n4 - 1) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (i4 * 4 + e >= n) u[e] = 0u;
  }
}

struct TopkShared {
  uint32_t hist[kTopkBins];
  uint32_t cand[kCandCap];
  uint32_t red[kTopkWarps], red2[kTopkWarps];
  uint32_t warp_gt[kTopkWarps], warp_eq[kTopkWarps], list_len[kTopkWarps];
  uint32_t digit, remaining;
};

// Bin d of sh.hist with  count(bins > d) < r <= count(bins >= d)  (1 <= r <= total); every thread gets d and
// r - count(bins > d).  All threads of the CTA call it, after a barrier that completed the histogram; one warp
// does the search (16 bins per lane) - the per-row costs of this kernel are instructions, and sixteen warps
// searching together would issue ten times as many.
__device__ __forceinline__ void find_bin(TopkShared& sh, uint32_t r, uint32_t& digit, uint32_t& rest) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp == 0) {
    constexpr int kPer = kTopkBins / 32;
    uint32_t c[kPer], ssum = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) { c[i] = sh.hist[lane * kPer + i]; ssum += c[i]; }
    uint32_t suf = ssum;                                 // sum over lanes >= lane
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t v = __shfl_down_sync(0xFFFFFFFFu, suf, off);
      if (lane + off < 32) suf += v;
    }
    const uint32_t above = suf - ssum;                   // in the bins of higher lanes
    if (above < r && r <= above + ssum) {
      uint32_t acc = above;
#pragma unroll
      for (int i = kPer - 1; i >= 0; --i) {
        if (acc < r && acc + c[i] >= r) {
          sh.digit = (uint32_t)(lane * kPer + i);
          sh.remaining = r - acc;
        }
        acc += c[i];
      }
    }
  }
  __syncthreads();
  digit = sh.digit;
  rest = sh.remaining;
  __syncthreads();
}

// sum / minimum / maximum over the 16 per-warp values of an array in shared memory: one load per lane and four
// shuffles instead of sixteen loads per thread
__device__ __forceinline__ uint32_t warps_sum(const uint32_t* a) {
  uint32_t v = a[threadIdx.x & (kTopkWarps - 1)];
#pragma unroll
  for (int off = kTopkWarps / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
  return v;
}
__device__ __forceinline__ uint32_t warps_min(const uint32_t* a) {
  uint32_t v = a[threadIdx.x & (kTopkWarps - 1)];
#pragma unroll
  for (int off = kTopkWarps / 2; off > 0; off >>= 1) v = min(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
  return v;
}
__device__ __forceinline__ uint32_t warps_max(const uint32_t* a) {
  uint32_t v = a[threadIdx.x & (kTopkWarps - 1)];
#pragma unroll
  for (int off = kTopkWarps / 2; off > 0; off >>= 1) v = max(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
  return v;
}
__device__ __forceinline__ uint32_t block_sum(TopkShared& sh, uint32_t v) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
  if (lane == 0) sh.red[warp] = v;
  __syncthreads();
  const uint32_t t = warps_sum(sh.red);
  __syncthreads();
  return t;
}

#ifndef KB200_TOPK_MIN_CTAS
#define KB200_TOPK_MIN_CTAS 2      // CTAs per SM the register allocation aims at (3, with a few spills, measured no faster)
#endif
__global__ void __launch_bounds__(kTopkThreads, KB200_TOPK_MIN_CTAS)
topk_select_kernel(const float* __restrict__ scores, int64_t row_stride, int n_cols,
                   const int32_t* __restrict__ n_valid, const int32_t* __restrict__ k_row, int k_max,
                   int32_t* __restrict__ out_idx, int64_t idx_stride, int32_t* __restrict__ out_count,
                   int64_t rows) {
  __shared__ TopkShared sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    int n = n_valid ? n_valid[row] : n_cols;
    n = max(0, min(n, n_cols));
    int k = k_row ? min(k_row[row], k_max) : k_max;
    k = max(0, min(k, n));
    int32_t* out = out_idx + row * idx_stride;
    if (tid == 0 && out_count) out_count[row] = k;
    if (k == 0) continue;
    if (k == n) {  // every candidate is selected
      for (int i = tid; i < n; i += kTopkThreads) out[i] = i;
      continue;
    }
    const float4* row4 = reinterpret_cast<const float4*>(scores + row * row_stride);
    const int n4 = (n + 3) >> 2;
    // warp w owns the 16-byte pieces [w_begin, w_end) of the row
    const int seg4 = (n4 + kTopkWarps - 1) / kTopkWarps;
    const int w_begin = min(warp * seg4, n4), w_end = min(w_begin + seg4, n4);
    const int w_iters = (w_end - w_begin + 31) >> 5;

    // ---- 1. bracket [lo_key, hi_key] of the k-th largest key from a sample ----------------------------
    // Two histogram levels: 512 bins over the sample's key range, then 512 bins over the few bins the two
    // ranks fell into - scores of a row often sit in a narrow band far below the row's maximum, and the first
    // level alone would cut that band into a dozen bins.
    uint32_t lo_key = 0u, hi_key = 0xFFFFFFFFu;
    const bool sampled = n > kListRow;
    if (sampled) {
      const int f4 = n > 65536 ? 4 : 2;                  // 16-byte pieces per thread: 4096 or 8192 sampled scores
      const int n_samp = f4 * kTopkThreads * 4;
      uint32_t sk[16], smin = 0xFFFFFFFFu, smax = 0u;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        if (it < f4) {
          const int pos = (int)(((int64_t)(it * kTopkThreads + tid) * n4) >> (f4 == 4 ? 11 : 10));  // < n4 - 1
          const float4 x = __ldg(row4 + pos);
          sk[it * 4 + 0] = float_key(x.x); sk[it * 4 + 1] = float_key(x.y);
          sk[it * 4 + 2] = float_key(x.z); sk[it * 4 + 3] = float_key(x.w);
        } else {
          sk[it * 4 + 0] = sk[it * 4 + 1] = sk[it * 4 + 2] = sk[it * 4 + 3] = sk[0];
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) { smin = min(smin, sk[i]); smax = max(smax, sk[i]); }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        smin = min(smin, __shfl_xor_sync(0xFFFFFFFFu, smin, off));
        smax = max(smax, __shfl_xor_sync(0xFFFFFFFFu, smax, off));
      }
      if (lane == 0) { sh.red[warp] = smin; sh.red2[warp] = smax; }
      for (int i = tid; i < kTopkBins; i += kTopkThreads) sh.hist[i] = 0;
      __syncthreads();
      const uint32_t bottom = warps_min(sh.red), top = warps_max(sh.red2);
      const float ks = (float)k * (float)n_samp / (float)n;                          // sample rank of the threshold
      const float margin = 5.f * sqrtf(ks) + 16.f;
      int r_hi = (int)(ks - margin), r_lo = (int)(ks + margin) + 1;                  // ranks from the top, 1-based
      // level 1
      uint32_t z_lo = bottom, z_hi = top, above = 0;     // zoom window and the samples above it
      {
        const uint32_t range = top - bottom;
        const int shift = (range >> kDigit) ? (32 - __clz(range) - kDigit) : 0;      // (range >> shift) < kTopkBins
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&sh.hist[(sk[i] - bottom) >> shift], 1u);
        if (f4 == 4) {
#pragma unroll
          for (int i = 8; i < 16; ++i) atomicAdd(&sh.hist[(sk[i] - bottom) >> shift], 1u);
        }
        __syncthreads();
        uint32_t b, rest;
        if (r_hi >= 1) {
          find_bin(sh, (uint32_t)r_hi, b, rest);
          above = (uint32_t)r_hi - rest;                                             // samples in the bins above b
          const uint64_t edge = (uint64_t)bottom + ((uint64_t)(b + 1) << shift);      // first key above bin b
          if (edge - 1 < (uint64_t)top) z_hi = (uint32_t)(edge - 1);
        }
        if (r_lo <= n_samp) {
          find_bin(sh, (uint32_t)r_lo, b, rest);
          z_lo = bottom + (b << shift);
        }
      }
      // level 2: the samples inside [z_lo, z_hi]
      {
        const uint32_t range = z_hi - z_lo;
        const int shift = (range >> kDigit) ? (32 - __clz(range) - kDigit) : 0;
        for (int i = tid; i < kTopkBins; i += kTopkThreads) sh.hist[i] = 0;
        __syncthreads();
        uint32_t inside = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (sk[i] - z_lo <= range) {                     // z_lo <= key <= z_hi
            atomicAdd(&sh.hist[(sk[i] - z_lo) >> shift], 1u);
            ++inside;
          }
        }
        if (f4 == 4) {
#pragma unroll
          for (int i = 8; i < 16; ++i) {
            if (sk[i] - z_lo <= range) {
              atomicAdd(&sh.hist[(sk[i] - z_lo) >> shift], 1u);
              ++inside;
            }
          }
        }
        const uint32_t n_inside = block_sum(sh, inside);  // (its barriers also publish the histogram)
        r_hi -= (int)above;
        r_lo -= (int)above;
        uint32_t b, rest;
        if (r_hi >= 1 && (uint32_t)r_hi <= n_inside) {    // keys above the bin of rank r_hi: (very likely) all selected
          find_bin(sh, (uint32_t)r_hi, b, rest);
          const uint64_t edge = (uint64_t)z_lo + ((uint64_t)(b + 1) << shift);
          hi_key = edge - 1 < (uint64_t)z_hi ? (uint32_t)(edge - 1) : z_hi;
        } else if (r_hi >= 1) {
          hi_key = z_hi;
        }
        if (r_lo >= 1 && (uint32_t)r_lo <= n_inside) {    // keys below the bin of rank r_lo: (very likely) none selected
          find_bin(sh, (uint32_t)r_lo, b, rest);
          lo_key = z_lo + (b << shift);
        } else if (r_lo > (int)n_inside && r_lo + (int)above <= n_samp) {
          lo_key = z_lo;
        }
      }
      if (hi_key < lo_key) { lo_key = 0u; hi_key = 0xFFFFFFFFu; }
    }

    // ---- 2. count the keys above hi_key, collect those in [lo_key, hi_key] --------------------------------
    // Every warp walks its own piece of the row and appends to a list of its own, so that nothing is shared
    // (one counter for the whole CTA would serialise a thousand atomics per row), and so that the list later
    // tells the warp how many of its scores lie above / at the threshold.
    lo_key = max(lo_key, 1u);
    uint32_t cnt_gt = 0, my_cand = 0;                     // my_cand: entries in this warp's list (warp-uniform)
    uint32_t* const my_list = sh.cand + warp * kWarpList;
    {
      for (int it0 = 0; it0 < w_iters; it0 += kTopkUnroll) {
        float4 xs[kTopkUnroll];                           // several loads in flight per lane
#pragma unroll
        for (int j = 0; j < kTopkUnroll; ++j) {
          const int i4 = w_begin + (it0 + j) * 32 + lane;
          xs[j] = i4 < w_end ? __ldg(row4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < kTopkUnroll; ++j) {
          if (it0 + j >= w_iters) break;                  // (the same for the whole warp)
          const int i4 = w_begin + (it0 + j) * 32 + lane;
          uint32_t u[4];
          piece_keys(xs[j], i4 < w_end ? i4 : n4, n4, n, u);
          bool cand[4];
          uint32_t c = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const bool gt = u[e] > hi_key;
            cand[e] = !gt && u[e] >= lo_key;
            cnt_gt += gt;
            c += cand[e];
          }
          if (__any_sync(0xFFFFFFFFu, c != 0)) {
            uint32_t incl = c;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
              const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
              if (lane >= off) incl += v;
            }
            uint32_t pos = my_cand + incl - c;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (cand[e]) {
                if (pos < (uint32_t)kWarpList) my_list[pos] = u[e];
                ++pos;
              }
            }
            my_cand += __shfl_sync(0xFFFFFFFFu, incl, 31);
          }
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) cnt_gt += __shfl_xor_sync(0xFFFFFFFFu, cnt_gt, off);
    const uint32_t my_gt_hi = cnt_gt;                     // scores of this warp's piece above hi_key
    if (lane != 0) cnt_gt = 0;
    if (lane == 0) sh.list_len[warp] = my_cand;
    const uint32_t n_gt = block_sum(sh, cnt_gt);          // (its barriers also publish the lists and their lengths)
    const uint32_t n_cand = warps_sum(sh.list_len);
    const bool fits = warps_max(sh.list_len) <= (uint32_t)kWarpList;

    if (!sampled) {
      // the whole row is the list: its own key range instead of all 32 bits, so that the first digit spreads
      uint32_t cmin = 0xFFFFFFFFu, cmax = 0u;
      if (fits)
        for (uint32_t i = lane; i < my_cand; i += 32) { cmin = min(cmin, my_list[i]); cmax = max(cmax, my_list[i]); }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        cmin = min(cmin, __shfl_xor_sync(0xFFFFFFFFu, cmin, off));
        cmax = max(cmax, __shfl_xor_sync(0xFFFFFFFFu, cmax, off));
      }
      if (lane == 0) { sh.red[warp] = cmin; sh.red2[warp] = cmax; }
      __syncthreads();
      cmin = warps_min(sh.red);
      cmax = warps_max(sh.red2);
      __syncthreads();
      lo_key = cmin;
      hi_key = cmax;
    }
    uint32_t tau = 0, need_eq = 0;
    if (fits && n_gt < (uint32_t)k && (uint32_t)k <= n_gt + n_cand) {
      // ---- the k-th largest key is the (k - n_gt)-th largest of the list --------------------------------
      const uint32_t range = hi_key - lo_key;
      const int nb = range ? 32 - __clz(range) : 0;
      uint32_t prefix = 0, mask = 0, remaining = (uint32_t)k - n_gt;
#pragma unroll 1
      for (int hb = nb; hb > 0; hb -= kDigit) {
        const int shift = max(hb - kDigit, 0);
        const uint32_t dmask = (1u << (hb - shift)) - 1u;
        for (int i = tid; i < kTopkBins; i += kTopkThreads) sh.hist[i] = 0;
        __syncthreads();
        for (uint32_t i = lane; i < my_cand; i += 32) {    // every warp bins its own list
          const uint32_t v = my_list[i] - lo_key;
          if ((v & mask) == prefix) atomicAdd(&sh.hist[(v >> shift) & dmask], 1u);
        }
        __syncthreads();
        uint32_t d;
        find_bin(sh, remaining, d, remaining);
        prefix |= d << shift;
        mask |= dmask << shift;
      }
      tau = lo_key + prefix;
      need_eq = remaining;
      // this warp's scores above / at the threshold: those above hi_key, and what its own list says
      uint32_t g = 0, q = 0;
      for (uint32_t i = lane; i < my_cand; i += 32) {
        const uint32_t v = my_list[i];
        g += v > tau;
        q += v == tau;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        g += __shfl_xor_sync(0xFFFFFFFFu, g, off);
        q += __shfl_xor_sync(0xFFFFFFFFu, q, off);
      }
      if (lane == 0) { sh.warp_gt[warp] = my_gt_hi + g; sh.warp_eq[warp] = q; }
    } else {
      // ---- 3. the sample misjudged the row: four histogram passes over the row itself -------------------
      const int iters = (n4 + kTopkThreads - 1) / kTopkThreads;
      uint32_t prefix = 0, mask = 0, remaining = (uint32_t)k;
#pragma unroll 1
      for (int hb = 32; hb > 0; hb -= kDigit) {
        const int shift = max(hb - kDigit, 0);
        const uint32_t dmask = (1u << (hb - shift)) - 1u;
        for (int i = tid; i < kTopkBins; i += kTopkThreads) sh.hist[i] = 0;
        __syncthreads();
        for (int it = 0; it < iters; ++it) {
          const int i4 = it * kTopkThreads + tid;
          const float4 x = i4 < n4 ? __ldg(row4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
          uint32_t u[4];
          piece_keys(x, i4 < n4 ? i4 : n4, n4, n, u);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const bool valid = u[e] != 0u && ((u[e] & mask) == prefix);
            const uint32_t digit = (u[e] >> shift) & dmask;
            // equal digits are common here (that is why the sample failed): aggregate within the warp
            const uint32_t peers = __match_any_sync(0xFFFFFFFFu, valid ? digit : 0xFFFFu);
            if (valid && (__ffs(peers) - 1) == lane) atomicAdd(&sh.hist[digit], (uint32_t)__popc(peers));
          }
        }
        __syncthreads();
        uint32_t d;
        find_bin(sh, remaining, d, remaining);
        prefix |= d << shift;
        mask |= dmask << shift;
      }
      tau = prefix;
      need_eq = remaining;
      // per warp: scores above / equal to the threshold in its piece (one more pass over the row)
      {
        uint32_t g = 0, q = 0;
        for (int it0 = 0; it0 < w_iters; it0 += kTopkUnroll) {
          float4 xs[kTopkUnroll];
  #pragma unroll
          for (int j = 0; j < kTopkUnroll; ++j) {
            const int i4 = w_begin + (it0 + j) * 32 + lane;
            xs[j] = i4 < w_end ? __ldg(row4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
  #pragma unroll
          for (int j = 0; j < kTopkUnroll; ++j) {
            const int i4 = w_begin + (it0 + j) * 32 + lane;
            const bool in = i4 < w_end;
            const uint32_t u[4] = {float_key(xs[j].x), float_key(xs[j].y), float_key(xs[j].z), float_key(xs[j].w)};
  #pragma unroll
            for (int e = 0; e < 4; ++e) {
              const bool ok = in && (i4 * 4 + e < n);
              g += ok && u[e] > tau;
              q += ok && u[e] == tau;
            }
          }
        }
  #pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          g += __shfl_xor_sync(0xFFFFFFFFu, g, off);
          q += __shfl_xor_sync(0xFFFFFFFFu, q, off);
        }
        if (lane == 0) { sh.warp_gt[warp] = g; sh.warp_eq[warp] = q; }
      }
    }
    // tau = key of the k-th largest score; `need_eq` keys equal to it are wanted, the lowest positions first

    __syncthreads();
    uint32_t gt_before, eq_before;                        // in the pieces of the warps before this one
    {
      const int w = lane & (kTopkWarps - 1);
      uint32_t g = w < warp ? sh.warp_gt[w] : 0u, q = w < warp ? sh.warp_eq[w] : 0u;
#pragma unroll
      for (int off = kTopkWarps / 2; off > 0; off >>= 1) {
        g += __shfl_xor_sync(0xFFFFFFFFu, g, off);
        q += __shfl_xor_sync(0xFFFFFFFFu, q, off);
      }
      gt_before = g;
      eq_before = q;
    }
    // ---- 4. write the selected positions of this warp's piece, in index order -----------------------------
    for (int it0 = 0; it0 < w_iters; it0 += kTopkUnroll) {
      float4 xs[kTopkUnroll];
#pragma unroll
      for (int j = 0; j < kTopkUnroll; ++j) {
        const int i4 = w_begin + (it0 + j) * 32 + lane;
        xs[j] = i4 < w_end ? __ldg(row4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < kTopkUnroll; ++j) {
        if (it0 + j >= w_iters) break;                    // (the same for the whole warp)
        const int i4 = w_begin + (it0 + j) * 32 + lane;
        uint32_t u[4];
        piece_keys(xs[j], i4 < w_end ? i4 : n4, n4, n, u);
        uint32_t gt[4], packed = 0;
        bool any_eq = false;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          gt[e] = u[e] > tau;
          packed += gt[e];
          any_eq |= u[e] == tau;
        }
        if (!__any_sync(0xFFFFFFFFu, any_eq)) {
          // no score at the threshold among these 128: positions follow from the counts of the lanes before
          uint32_t incl = packed;
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
            if (lane >= off) incl += v;
          }
          uint32_t at = gt_before + min(eq_before, need_eq) + incl - packed;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (gt[e]) out[at++] = i4 * 4 + e;
          }
          gt_before += __shfl_sync(0xFFFFFFFFu, incl, 31);
        } else {
          uint32_t eq[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            eq[e] = u[e] == tau;
            packed += eq[e] << 16;
          }
          uint32_t incl = packed;                          // (eq << 16 | gt) of the lanes up to this one
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) {
            const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
            if (lane >= off) incl += v;
          }
          const uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31);
          const uint32_t excl = incl - packed;
          uint32_t g0 = gt_before + (excl & 0xFFFFu), q0 = eq_before + (excl >> 16);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const bool sel = gt[e] || (eq[e] && q0 < need_eq);
            if (sel) out[g0 + min(q0, need_eq)] = i4 * 4 + e;
            g0 += gt[e];
            q0 += eq[e];
          }
          gt_before += total & 0xFFFFu;
          eq_before += total >> 16;
        }
      }
    }
    __syncthreads();                                      // the shared arrays are reused by the next row
  }
}

__global__ void prefill_budgets_kernel(int32_t* n_valid, int32_t* k_row, int num_tiles, int total,
                                       int k_max, float pct, int rolling) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int t = i % num_tiles;
  int start = t * kTile;
  n_valid[i] = start;
  int k = k_max;
  if (rolling) {
    // strategies/KascadeStrategy.py:137: (pct * tile_start) // 100, at least 128
    int r = (int)floor((double)pct * (double)start / 100.0);
    k = min(k_max, max(128, r));
  }
  k_row[i] = k;
}

// per-sequence budgets of a ragged batch: the reference's formulas for a prompt of seq_len[b] tokens
// (strategies/KascadeStrategy.py:127-139); tiles beyond a sequence's end get no candidates
__global__ void prefill_budgets_ragged_kernel(int32_t* n_valid, int32_t* k_row, const int32_t* seq_len, int groups,
                                              int num_tiles, int total, int k_cap, float pct, int rolling) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int t = i % num_tiles, b = i / (num_tiles * groups);
  const int L = max(seq_len[b], 0), start = t * kTile;
  int kk = min(max(128, (int)((double)pct / 100.0 * (double)L)), L) - kTile;
  kk = max(kk, 0);
  int k = kk;
  if (rolling && L > 128) {
    int r = (int)floor((double)pct * (double)start / 100.0);
    k = min(kk, max(128, r));
  }
  const bool live = start < L;
  n_valid[i] = live ? start : 0;
  k_row[i] = live ? min(k, k_cap) : 0;
}

}  // namespace kb200

extern "C" int kb200_prefill_budgets_ragged(int32_t* n_valid, int32_t* k_row, const int32_t* seq_len, int batch,
                                            int num_kv_heads, int num_tiles, int k_cap, float pct, int rolling,
                                            void* stream) {
  using namespace kb200;
  KB_ENTRY(n_valid, "prefill_budgets_ragged: n_valid");
  KB_REQUIRE(n_valid && k_row && seq_len, "prefill_budgets_ragged: null pointer");
  int total = batch * num_kv_heads * num_tiles;
  if (total <= 0) return 0;
  prefill_budgets_ragged_kernel<<<ceil_div(total, 256), 256, 0, (cudaStream_t)stream>>>(
      n_valid, k_row, seq_len, num_kv_heads, num_tiles, total, k_cap, pct, rolling);
  KB_CHECK_LAUNCH("prefill_budgets_ragged_kernel");
  return 0;
}

extern "C" int kb200_topk_select(const float* scores, int64_t row_stride, int n_cols,
                                 const int32_t* n_valid, const int32_t* k_row, int k_max,
                                 int32_t* out_idx, int64_t idx_stride, int32_t* out_count,
                                 int64_t rows, void* stream) {
  using namespace kb200;
  KB_ENTRY(scores, "topk_select: scores");
  KB_REQUIRE(scores && out_idx, "topk_select: null pointer");
  KB_REQUIRE(rows >= 0 && n_cols >= 0 && k_max >= 0, "topk_select: negative size");
  KB_REQUIRE(n_cols <= row_stride, "topk_select: n_cols (%d) exceeds row_stride (%lld)", n_cols,
             (long long)row_stride);
  KB_REQUIRE(row_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(scores) & 15) == 0,
             "topk_select: rows must be 16-byte aligned (row_stride %% 4 == 0)");
  KB_REQUIRE(idx_stride >= (int64_t)k_max, "topk_select: idx_stride (%lld) smaller than k_max (%d)",
             (long long)idx_stride, k_max);
  if (rows == 0) return 0;
  int64_t grid = rows < (int64_t)sm_count() * 64 ? rows : (int64_t)sm_count() * 64;
  topk_select_kernel<<<(unsigned)grid, kTopkThreads, 0, (cudaStream_t)stream>>>(
      scores, row_stride, n_cols, n_valid, k_row, k_max, out_idx, idx_stride, out_count, rows);
  KB_CHECK_LAUNCH("topk_select_kernel");
  return 0;
}

extern "C" int kb200_prefill_budgets(int32_t* n_valid, int32_t* k_row, int batch, int num_kv_heads,
                                     int num_tiles, int k_max, float pct, int rolling, void* stream) {
  using namespace kb200;
  KB_ENTRY(n_valid, "prefill_budgets: n_valid");
  KB_REQUIRE(n_valid && k_row, "prefill_budgets: null pointer");
  int total = batch * num_kv_heads * num_tiles;
  if (total <= 0) return 0;
  prefill_budgets_kernel<<<ceil_div(total, 256), 256, 0, (cudaStream_t)stream>>>(
      n_valid, k_row, num_tiles, total, k_max, pct, rolling);
  KB_CHECK_LAUNCH("prefill_budgets_kernel");
  return 0;
}
