// Exact per-row Top-k by radix select (one CTA per row).
//
// Replaces the torch.topk call sites of the reference's efficient path
// (strategies/EfficientKascadeStrategy.py:82,90,111).  The row is read from global memory (L2 after
// the first pass): three 11/11/10-bit histogram passes find the k-th largest key exactly, a fourth pass
// compacts the selected positions in ascending index order, taking ties at the threshold from the
// lowest index upwards.
#include "common.cuh"

namespace kb200 {

constexpr int kTopkThreads = 512;
constexpr int kTopkBins = 2048;                           // 11-bit digits: 3 passes cover the 32-bit key

// order-preserving map float -> uint32 (larger float <=> larger key)
__device__ __forceinline__ uint32_t float_key(float x) {
  uint32_t b = __float_as_uint(x);
  return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}

__global__ void __launch_bounds__(kTopkThreads)
topk_select_kernel(const float* __restrict__ scores, int64_t row_stride, int n_cols,
                   const int32_t* __restrict__ n_valid, const int32_t* __restrict__ k_row, int k_max,
                   int32_t* __restrict__ out_idx, int64_t idx_stride, int32_t* __restrict__ out_count,
                   int64_t rows) {
  __shared__ uint32_t hist[kTopkBins];
  __shared__ uint32_t warp_tot[kTopkThreads / 32];
  __shared__ uint32_t sh_digit, sh_remaining;
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
    const int iters = (n4 + kTopkThreads - 1) / kTopkThreads;

    // three histogram passes over key bits [31:21], [20:10], [9:0]; post-softmax scores spread over
    // many exponent / mantissa bins in every pass, so plain shared-memory atomics do
    uint32_t prefix = 0, mask = 0, remaining = (uint32_t)k;
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
      const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
      const uint32_t dmask = pass == 2 ? 1023u : 2047u;
      for (int i = tid; i < kTopkBins; i += kTopkThreads) hist[i] = 0;
      __syncthreads();
      for (int it = 0; it < iters; ++it) {
        const int i4 = it * kTopkThreads + tid;
        const bool in = i4 < n4;
        const float4 x = in ? __ldg(row4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t u = float_key(xs[e]);
          const bool valid = in && (i4 * 4 + e < n) && ((u & mask) == prefix);
          const uint32_t digit = (u >> shift) & dmask;
          if (pass == 0) {
            // the leading bits of the scores of a row mostly coincide: aggregate within the warp
            const uint32_t peers = __match_any_sync(0xFFFFFFFFu, valid ? digit : 0xFFFFu);
            if (valid && (__ffs(peers) - 1) == lane) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
          } else if (valid) {
            atomicAdd(&hist[digit], 1u);
          }
        }
      }
      __syncthreads();
      // bin d with count(> d) < remaining <= count(>= d): suffix sums over 4 bins per thread
      {
        uint32_t c[4], ssum = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) { c[i] = hist[tid * 4 + i]; ssum += c[i]; }
        uint32_t suf = ssum;                               // sum over lanes >= lane of this warp
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const uint32_t v = __shfl_down_sync(0xFFFFFFFFu, suf, off);
          if (lane + off < 32) suf += v;
        }
        if (lane == 0) warp_tot[warp] = suf;
        __syncthreads();
        uint32_t higher = 0;
#pragma unroll
        for (int w = 0; w < kTopkThreads / 32; ++w) higher += w > warp ? warp_tot[w] : 0u;
        const uint32_t above = higher + suf - ssum;        // candidates in bins of higher threads
        if (above < remaining && remaining <= above + ssum) {
          uint32_t acc = above;
#pragma unroll
          for (int i = 3; i >= 0; --i) {
            if (acc < remaining && acc + c[i] >= remaining) {
              sh_digit = (uint32_t)(tid * 4 + i);
              sh_remaining = remaining - acc;
            }
            acc += c[i];
          }
        }
      }
      __syncthreads();
      prefix |= sh_digit << shift;
      mask |= dmask << shift;
      remaining = sh_remaining;
      __syncthreads();
    }
    // prefix = key of the k-th largest score; `remaining` keys equal to it are still wanted
    const uint32_t tau = prefix, need_eq = remaining;
    uint32_t gt_total = 0, eq_total = 0;
    for (int it = 0; it < iters; ++it) {
      int i4 = it * kTopkThreads + tid;
      bool in = i4 < n4;
      float4 x = in ? __ldg(row4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
      float xs[4] = {x.x, x.y, x.z, x.w};
      uint32_t gt[4], eq[4], packed = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t u = float_key(xs[e]);
        bool ok = in && (i4 * 4 + e < n);
        gt[e] = ok && (u > tau);
        eq[e] = ok && (u == tau);
        packed += gt[e] + (eq[e] << 16);
      }
      // block-wide exclusive scan of (eq << 16 | gt) in index order
      uint32_t incl = packed;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if (lane >= off) incl += v;
      }
      if (lane == 31) warp_tot[warp] = incl;
      __syncthreads();
      uint32_t base = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kTopkThreads / 32; ++w) {
        uint32_t v = warp_tot[w];
        if (w < warp) base += v;
        total += v;
      }
      uint32_t excl = base + incl - packed;
      uint32_t gt_before = gt_total + (excl & 0xFFFFu);
      uint32_t eq_before = eq_total + (excl >> 16);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        bool sel = gt[e] || (eq[e] && eq_before < need_eq);
        if (sel) out[gt_before + min(eq_before, need_eq)] = i4 * 4 + e;
        gt_before += gt[e];
        eq_before += eq[e];
      }
      gt_total += total & 0xFFFFu;
      eq_total += total >> 16;
      __syncthreads();
    }
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
