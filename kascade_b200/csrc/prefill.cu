// Tile prefill kernels on the sm_100a tensor-core path (tcgen05.mma, accumulators in tensor memory).
//
// A work item is one query tile: 32 consecutive queries x the 4 query heads of one KV head = 128
// rows (row = 4 * query_in_tile + head), the M dimension of every MMA.  Keys arrive in blocks of
// 128 rows.  The same kernel body serves four modes:
//
//   kDenseAttn  causal attention over keys 0 .. last query of the tile; writes O and lse2
//               (replaces `prefill`, kernels/flash_attention/recompute_kascade_gqa_prefill.py:224-274)
//   kDenseLse   the same without V: lse2 only
//               (replaces `compute_scores`, recompute_kascade_gqa_prefill.py:276-312)
//   kSparse     keys = the tile's selected index row followed by the tile's own keys
//               (replaces `main_kernel`, kernels/flash_attention/reuse_kascade_gqa_prefill.py:146-198)
//   kPool       S^T = K_block . Q_tile^T so that tensor-memory lanes are keys; each reducer thread
//               sums exp2(s * scale2 - lse2[row]) over the 128 rows of the tile for its key
//               (replaces `aggregate`, recompute_kascade_gqa_prefill.py:171-222)
//
// The kernels are persistent: one CTA per SM walks the list of tiles (ordered by descending cost,
// handed out boustrophedon-wise), ring stages and barrier phases keep counting across tiles, so the
// next tile's Q/K/V are already on their way while the current tile is being finished.
//
// Warp roles (whole warps run their role with uniform control flow; one elected lane issues MMAs).
//   with V, dense (384 threads):  warps 0-7 two softmax warpgroups (key blocks j = w mod 2, thread =
//     tensor-memory lane = row); warp 8 lane 0 TMA box copies of Q and the K ring, warp 10 lane 0 of the
//     V ring (4-D tiled tensor maps, 128-byte swizzle, no multicast); warp 9 issues Q.K^T, warp 11 P.V.
//   with V, sparse (512 threads): warps 8-10 gather the selected K rows and warps 11, 14, 15 the V rows
//     with cp.async (16-byte chunks, 16 lanes per 256-byte row, written directly in the
//     128-byte-swizzled operand layout of umma.cuh); warp 12 issues Q.K^T, warp 13 P.V.
//   without V (512 threads):      warps 0-11 three softmax / reducer warpgroups (key blocks j = w mod 3);
//     warp 12 lane 0 TMA copies, warp 13 issues Q.K^T.
// setmaxnreg moves registers from the producer / MMA warpgroups to the softmax warpgroups.
// Hand-offs are mbarriers; every wait is bounded (umma::mbar_wait) and a kernel that gives up
// records a code in the device status word, drains its copies, frees its tensor memory and returns.
//
// Tensor memory (512 columns).  With V: S0 [0,128), S1 [128,256), P0 [256,320), P1 [320,384) (fp16 pairs,
// the A operand of P.V), O [384,512) - one accumulator for both streams, see the softmax role.
// Without V: S0, S1, S2.
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>
#include <atomic>
#include <mutex>

#include <cuda_bf16.h>

#include "common.cuh"
#include "umma.cuh"

namespace kb200 {

enum PrefillMode { kDenseAttn = 0, kDenseLse = 1, kSparse = 2, kPool = 3 };

constexpr int kStageBytes = 128 * kD * 2;     // one 128-row operand tile (32 KB)
constexpr int kNKMax = 6;                     // K ring: 3 stages with a V ring, 6 without
constexpr int kNV = 3;
constexpr float kRescaleLog2 = 8.0f;          // see the softmax role
constexpr int kPadAllowance = 512;            // tiles need 1024-byte alignment

__device__ int g_status_word = 0;

struct PrefillParams {
  const __half* q; int64_t q_sb, q_st, q_sh;
  const __half* k; int64_t k_sb, k_st, k_sh;
  const __half* v; int64_t v_sb, v_st, v_sh;
  const int32_t* tile_idx; int64_t idx_stride;
  const int32_t* tile_count;
  const int32_t* head_map;
  float scale2;
  int bf16;                       // host side: the activations (and the outputs) are bf16, not fp16
  __half* out;                    // == out_fan[0] unless the output goes to several GPUs
  __half* out_fan[KB200_MAX_FANOUT];   // outputs [B, L, H_out, D]: this GPU's own buffer and its peers'
  int n_fan, H_out, h_off;        // number of outputs, heads of an output row, first head written by this call
  int mc;                         // out_fan[0] is a multicast address: rows are stored with multimem.st
  float* lse2;
  const float* lse2_in;
  float* pooled; int64_t pooled_stride;
  int B, L, H, G, T;                  // L: tokens of a batch slot (the longest sequence), T: its tiles
  // Ragged batches (NULL: every sequence has L tokens starting at row 0 of its slot): sequence b occupies
  // rows seq_start[b] .. seq_start[b] + seq_len[b] - 1 of slot b; tiles beyond a sequence's end are skipped.
  const int32_t* seq_start;
  const int32_t* seq_len;
  int G_idx;                      // KV heads in the index tensors (>= G when heads are sharded)
  int group;                      // (sequence, KV head) pairs whose tiles are walked together, divides B * G
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
// 16-byte copy that writes zeros when src_bytes == 0 (the source address must still be valid)
__device__ __forceinline__ void cp16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
// the barrier receives one arrival from this thread once all its earlier cp.async have completed
__device__ __forceinline__ void cp_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(umma::smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
// 2^x on the FMA pipes, for x <= 127: the special-function unit delivers 16 results per clock and SM,
// which is what bounds the softmax; every fourth exponential goes this way instead.  x is rounded
// to the nearest integer n by adding 1.5 * 2^23 (n lands in the low mantissa bits), 2^(x - n) on
// [-0.5, 0.5] is a degree-4 polynomial (relative error 3e-6), and n is added to the exponent field.
// Share of the exponentials of the lse and pool passes that goes to the FMA pipes: every fourth one, and with
// EXTRA = n > 0 one more in every n-th group of four.  Measured at 32 768 tokens: the lse pass is fastest with
// a quarter (3/8: +11 %), the pool pass, whose other arithmetic is packed two per instruction, with 3/8 (-4 %).
#ifndef KB200_POLY_EXTRA_LSE
#define KB200_POLY_EXTRA_LSE 0
#endif
#ifndef KB200_POLY_EXTRA_POOL
#define KB200_POLY_EXTRA_POOL 2
#endif
template <int EXTRA>
__device__ __forceinline__ constexpr bool poly_also(int i) {
  return EXTRA > 0 && ((i >> 2) % (EXTRA > 0 ? EXTRA : 1)) == 0;
}
__device__ __forceinline__ float ex2_fma(float x) {
#ifdef KB200_NO_FMA_EXP
  return ex2(x);
#endif
  x = fmaxf(x, -120.0f);                               // also maps -inf (masked) to 2^-120 ~ 0
  const float t = x + 12582912.0f;
  const float f = x - (t - 12582912.0f);
  float q = 0.009585312567651272f;
  q = fmaf(q, f, 0.05590597912669182f);
  q = fmaf(q, f, 0.24024048447608948f);
  q = fmaf(q, f, 0.6931242942810059f);
  q = fmaf(q, f, 1.0f);
  return __uint_as_float(__float_as_uint(q) + (__float_as_uint(t) << 23));
}
// Two fp32 operations per instruction (sm_100: fma / add on register pairs) and the three-input maximum:
// the softmax warps are bound by the number of instructions they issue, not by a single pipe, so every
// per-element instruction that two elements can share is worth taking.  Results are those of the scalar
// forms, bit for bit.
__device__ __forceinline__ uint64_t pair_u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pair_f(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpair_f(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 16 bytes to an NVLink multicast address (the mapping of a multicast object): delivered to every GPU bound to it
__device__ __forceinline__ void multimem_st16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
// two fp32 values -> one 32-bit pair in the storage type of the activations (fp16, or bf16 when BF16)
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Barriers and small exchange buffers; lives in dynamic shared memory behind the operand tiles so that
// the 7 x 32 KB tiles, the alignment padding and this block together stay inside the 227 KB limit.
struct PfShared {
  uint64_t bar_q, bar_qempty, bar_kfull[kNKMax], bar_kempty[kNKMax], bar_vfull[kNV], bar_vempty[kNV];
  uint64_t bar_sfull[3], bar_pready[3], bar_odone[3], bar_x, bar_ofree, bar_lse[3], bar_sfree[2], bar_turn[2];
  uint32_t tmem;
  int give_up;
  int abort;                                           // copy of the device status word taken at CTA start
  union {
    float xchg[2][2][128];                             // softmax modes: [m (with V: row reference) | l][warpgroup][row]
    float lse[2][2][128];                              // pool mode: lse2 of the tile's rows [warpgroup][tile parity]
  };
};
static_assert(sizeof(PfShared) <= 2560, "PfShared grew");
constexpr int kSmemAttn = kStageBytes * (1 + 3 + kNV) + kPadAllowance + 2560;   // = 232448, the sm_100 limit
constexpr int kNKNoV = 5;                     // K ring of the modes without V
constexpr int kXchgNoV = 3 * 2 * 128 * 4;     // their exchange area behind PfShared: three streams x two values x 128 rows
constexpr int kSmemNoV = kStageBytes * (1 + kNKNoV) + kPadAllowance + 2560 + kXchgNoV;

// One work item = one query tile of one KV head of one sequence.
struct TileItem {
  int b, g, t, tile_start, rows_valid, count, total, nb;
  int L, row0;                          // tokens of this sequence, its first row inside the batch slot
  const int32_t* idx_row;
};

template <int MODE>
__device__ __forceinline__ TileItem decode_item(const PrefillParams& p, int item) {
  TileItem it;
  // items are ordered by descending tile index, i.e. by descending cost, so the boustrophedon
  // hand-out gives every CTA the same amount of work
  // The (sequence, KV head) pairs are taken `p.group` at a time: all tiles of one group before the
  // next, so that the K/V a group streams (group x L x 256 or 512 bytes) stay resident in L2 while
  // the CTAs sweep them; the host picks the group size from L (all pairs together for short prompts).
  const int per = p.group * p.T;
  const int hi = item / per, lo = item - hi * per;
  const int r = lo / p.group, bg = hi * p.group + (lo - r * p.group);
  it.t = p.T - 1 - r;
  it.b = bg / p.G;
  it.g = bg - it.b * p.G;
  it.tile_start = it.t * kTile;
  it.L = p.seq_len ? min(max(p.seq_len[it.b], 0), p.L) : p.L;
  it.row0 = p.seq_start ? p.seq_start[it.b] : 0;
  it.rows_valid = min(kTile, it.L - it.tile_start);
  it.count = 0;
  it.idx_row = nullptr;
  if (it.rows_valid <= 0) {                             // a tile beyond the end of a short sequence
    it.rows_valid = 0;
    it.total = 0;
  } else if (MODE == kSparse) {
    const int src_g = p.head_map ? p.head_map[it.g] : it.g;
    const int64_t row = ((int64_t)it.b * p.G_idx + src_g) * p.T + it.t;
    const int c = p.tile_count[row];
    it.count = max(0, min(c, (int)min((int64_t)it.tile_start, p.idx_stride)));
    it.idx_row = p.tile_idx + row * p.idx_stride;
    it.total = it.count + it.rows_valid;
  } else if (MODE == kPool) {
    it.total = it.tile_start;                          // keys strictly before the tile
  } else {
    it.total = it.tile_start + it.rows_valid;          // causal: keys up to the tile's last query
  }
  it.nb = (it.total + 127) >> 7;
  return it;
}

template <int MODE>
struct PfCfg {
  static constexpr bool kHasV = MODE == kDenseAttn || MODE == kSparse;
  static constexpr bool kIsPool = MODE == kPool;
  static constexpr bool kGather = MODE == kSparse;
  // softmax warpgroups (streams): two with V; three without V, where nothing but latency limits them
  static constexpr int kStreams = kHasV ? 2 : 3;
  static constexpr int kSoftmaxWarps = 4 * kStreams;
  // warps that issue Q.K^T without V: two taking the key blocks in turn paid off in the pool mode (-4 %),
  // not in the lse mode
  static constexpr int kIssuers = kIsPool ? 2 : 1;
  static constexpr int kThreads = (kGather || !kHasV) ? 512 : 384;
  static constexpr int kNK = kHasV ? 3 : kNKNoV;
  static constexpr int kProducerArrivals = 1;                   // Q tile: one thread announces the TMA bytes
  static constexpr int kRingArrivals = kGather ? 96 : 1;        // K / V stage: three gather warps each
  static constexpr int kProducerWarp0 = kHasV ? 8 : 12;
  static constexpr int kMmaWarp = kGather ? 12 : (kHasV ? 9 : 13);
};

template <int MODE, bool BF16>
__global__ void __launch_bounds__(PfCfg<MODE>::kThreads, 1)
tile_prefill_kernel(const __grid_constant__ PrefillParams p, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  using namespace umma;
  using Cfg = PfCfg<MODE>;
  constexpr bool HAS_V = Cfg::kHasV;
  constexpr bool POOL = Cfg::kIsPool;
  constexpr bool GATHER = Cfg::kGather;
  constexpr int kNK = Cfg::kNK;
  constexpr int kMmaWarp = Cfg::kMmaWarp;

  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t pad = (1024u - (smem_addr(smem_raw) & 1023u)) & 1023u;
  if (pad > (uint32_t)kPadAllowance) {                   // never seen; refuse rather than overrun
    if (tid == 0) atomicCAS(&g_status_word, 0, 90);
    return;
  }
  uint8_t* smem = smem_raw + pad;
  constexpr int kTiles = 1 + kNK + (HAS_V ? kNV : 0);
  PfShared& sh = *reinterpret_cast<PfShared*>(smem + kTiles * kStageBytes);
  // an earlier CTA or kernel gave up a bounded wait: do not queue up more waits behind it.  One thread
  // reads the word and the whole CTA takes the same decision.
  if (tid == 0) sh.abort = *reinterpret_cast<volatile int*>(&g_status_word);
  __syncthreads();
  if (sh.abort != 0) return;
  // modes without V: [3 streams][2][128] floats behind PfShared (partial row statistics / staged lse values)
  float* const xchg3 = reinterpret_cast<float*>(smem + kTiles * kStageBytes + 2560);
  uint64_t* bar_kfull = sh.bar_kfull;
  uint64_t* bar_kempty = sh.bar_kempty;
  uint64_t* bar_vfull = sh.bar_vfull;
  uint64_t* bar_vempty = sh.bar_vempty;
  uint64_t* bar_sfull = sh.bar_sfull;
  uint64_t* bar_pready = sh.bar_pready;
  uint64_t* bar_odone = sh.bar_odone;
  int& give_up = sh.give_up;
  const uint32_t q_s = smem_addr(smem);
  const uint32_t k_s = q_s + kStageBytes;
  const uint32_t v_s = k_s + kNK * kStageBytes;

  if (tid == 0) {
    mbar_init(&sh.bar_q, Cfg::kProducerArrivals);
    mbar_init(&sh.bar_qempty, HAS_V ? 1 : Cfg::kIssuers);   // one arrival per Q.K^T issuer
    mbar_init(&sh.bar_turn[0], 1);
    mbar_init(&sh.bar_turn[1], 1);
    for (int i = 0; i < kNK; ++i) { mbar_init(&bar_kfull[i], HAS_V ? Cfg::kRingArrivals : Cfg::kProducerArrivals); mbar_init(&bar_kempty[i], 1); }
    for (int i = 0; i < kNV; ++i) { mbar_init(&bar_vfull[i], Cfg::kRingArrivals); mbar_init(&bar_vempty[i], 1); }
    // each softmax warpgroup (128 threads) owns every other key block of a tile
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bar_sfull[i], 1);
      mbar_init(&bar_pready[i], 128);
      mbar_init(&bar_odone[i], 1);
    }
    for (int i = 0; i < 3; ++i) mbar_init(&sh.bar_lse[i], 128);
    for (int i = 0; i < 2; ++i) mbar_init(&sh.bar_sfree[i], 128);
    mbar_init(&sh.bar_x, Cfg::kSoftmaxWarps * 32);
    mbar_init(&sh.bar_ofree, Cfg::kSoftmaxWarps * 32);
    mbar_fence_init();
    give_up = 0;
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&sh.tmem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem;
  const uint32_t t_s0 = tmem;

  const int n_items = p.B * p.G * p.T;
  const int P = (int)gridDim.x;
  const int n_rounds = (n_items + P - 1) / P;
  auto item_of = [&](int k) -> int { return k * P + ((k & 1) ? (P - 1 - (int)blockIdx.x) : (int)blockIdx.x); };

  // ================================ producer: gathered rows by cp.async (sparse mode) ===========
  // Every thread copies with cp.async and lets the hardware arrive on the stage's "full" barrier when
  // its copies have landed (cp.async.mbarrier.arrive.noinc): the producers never wait for data, they
  // run ahead as far as the rings allow.  The MMA warps order the landed bytes against the tensor
  // core's reads with a proxy fence after their barrier waits.
  // One warp issues a 512-byte cp.async instruction only every ~50 cycles, however little else it
  // does, and the SM takes one about every 12: six warps gather, three per ring (rows 0-47, 48-95,
  // 96-127 of a stage), the K ring independent of the V ring.
  auto producer_gather = [&]() {
    const int gw = warp < 12 ? warp - 8 : warp - 10;     // warps 8, 9, 10: K ring; warps 11, 14, 15: V ring
    const bool is_v = gw >= 3;
    const int part = is_v ? gw - 3 : gw;
    const int r_begin = part * 48;                       // this warp's rows of a 128-row stage: 48, 48, 32
    const bool has_tail = part < 2;                      // rows r_begin + 32 .. r_begin + 47
    uint64_t* bar_full = is_v ? bar_vfull : bar_kfull;
    uint64_t* bar_empty = is_v ? bar_vempty : bar_kempty;
    const uint32_t ring_s = is_v ? v_s : k_s;
    const int n_st = is_v ? kNV : kNK;
    int st = 0, ph = 1;                                  // ring position, parity of its "empty" phase
    bool ok = true;
    uint32_t soff[4];                                    // swizzled offset of (row 2 q + (lane >> 4), chunk lane & 15)
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) soff[q4] = tile_off(2 * q4 + (lane >> 4), lane & 15, 128);
    const int sub = lane >> 4;
    const int tok_bytes = (int)((is_v ? p.v_st : p.k_st) * 2);   // host side checks that this fits
    // What the gather needs to know of a tile.  The next tile's record is fetched (two dependent global
    // loads: head map, row count) while the current tile is being gathered, and the index loads run two
    // key blocks ahead ACROSS the tile boundary, so the warps do not stall at the start of a tile.
    struct GatherTile {
      const char* base;                                  // this lane's 16-byte chunk of key 0 of the (sequence, KV head)
      const int32_t* idx;
      int count, total, tile_start, nb, L;
    };
    auto fetch = [&](int k) -> GatherTile {
      GatherTile g;
      g.base = nullptr; g.idx = nullptr; g.count = 0; g.total = 0; g.tile_start = 0; g.nb = 0; g.L = 1;
      if (k < n_rounds) {
        const int item = item_of(k);
        if (item < n_items) {
          const TileItem it = decode_item<MODE>(p, item);
          g.base = reinterpret_cast<const char*>(
              (is_v ? p.v + (int64_t)it.b * p.v_sb + (int64_t)it.row0 * p.v_st + (int64_t)it.g * p.v_sh
                    : p.k + (int64_t)it.b * p.k_sb + (int64_t)it.row0 * p.k_st + (int64_t)it.g * p.k_sh) + (lane & 15) * 8);
          g.idx = it.idx_row; g.count = it.count; g.total = it.total; g.tile_start = it.tile_start; g.nb = it.nb;
          g.L = it.L;
        }
      }
      return g;
    };
    // key position of row (r_begin + 32 r + lane) of key block j of tile g
    auto key_of = [&](const GatherTile& g, int j, int r) -> int {
      const int s = j * 128 + r_begin + r * 32 + lane;
      if (s >= g.total || (r == 1 && (!has_tail || lane >= 16))) return 0;
      return s < g.count ? __ldg(g.idx + s) : g.tile_start + (s - g.count);
    };
    GatherTile cur = fetch(0);
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;                  // keys of the next block and of the one after it
    bool a_ok = false, b_ok = false;
    for (int k = 0; k < n_rounds && ok; ++k) {
      const GatherTile nxt = fetch(k + 1);
      // The next tile's index row comes from HBM (every row is read once): pull it into L2 now, a whole
      // tile ahead, so that the index loads two blocks ahead of the copies find it there.  One warp per
      // ring does it; a lane touches every 32nd 128-byte line.
      if (part == 0 && nxt.idx != nullptr) {
        const char* row_bytes = reinterpret_cast<const char*>(nxt.idx);
        for (int off = lane * 128; off < nxt.count * 4; off += 32 * 128)
          asm volatile("prefetch.global.L2 [%0];\n" ::"l"(row_bytes + off));
      }
      for (int j = 0; j < cur.nb; ++j) {
        if (!a_ok) { a0 = key_of(cur, j, 0); a1 = key_of(cur, j, 1); }
        const int key0 = max(0, min(a0, cur.L - 1)), key1 = max(0, min(a1, cur.L - 1));
        a0 = b0; a1 = b1; a_ok = b_ok;
        const int j2 = j + 2;
        if (j2 < cur.nb) { b0 = key_of(cur, j2, 0); b1 = key_of(cur, j2, 1); b_ok = true; }
        else if (j2 - cur.nb < nxt.nb) { b0 = key_of(nxt, j2 - cur.nb, 0); b1 = key_of(nxt, j2 - cur.nb, 1); b_ok = true; }
        else b_ok = false;
        ok = mbar_wait(&bar_empty[st], ph, &give_up, is_v ? 12 : 11);
        if (!ok) break;
        // Per copy: one shuffle (the row's key), one multiply-add (its address), one cp.async; the
        // swizzled destination of row (2 i + sub) repeats every four i, 1024 bytes further on.
        const uint32_t dst = ring_s + st * kStageBytes + r_begin * 128;
        const char* base = cur.base;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int key = __shfl_sync(0xFFFFFFFFu, key0, i * 2 + sub);
          cp16(dst + (i >> 2) * 1024 + soff[i & 3], base + (int64_t)key * tok_bytes);
        }
        if (has_tail) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int key = __shfl_sync(0xFFFFFFFFu, key1, i * 2 + sub);
            cp16(dst + 4096 + (i >> 2) * 1024 + soff[i & 3], base + (int64_t)key * tok_bytes);
          }
        }
        cp_arrive_noinc(&bar_full[st]);
        if (++st == n_st) { st = 0; ph ^= 1; }
      }
      cur = nxt;
    }
    cp_wait_all();                                       // nothing of this CTA is in flight at teardown
  };

  // ================================ producer: TMA box copies (dense modes), one thread ===========
  // Tensor-map dimensions are (d, head, token, batch); a K/V tile is two boxes of 64 x 1 x 128 x 1 (the
  // two 64-column halves of the operand tile), a Q tile two boxes of 64 x 4 x 32 x 1 whose rows come
  // out as row = 4 * token + head.  Rows past the prompt are zero-filled by the copy engine.
  auto producer_tma = [&]() {                          // Q tiles and the K ring
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    int st = 0, ph = 1, qn = 0;
    bool ok = true;
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      if (it.nb == 0) continue;
      ok = mbar_wait(&sh.bar_qempty, (qn & 1) ^ 1, &give_up, 13);
      if (!ok) break;
      mbar_arrive_expect_tx(&sh.bar_q, kStageBytes);
      tma_load_4d(q_s, &tm_q, 0, it.g * kHg, it.row0 + it.tile_start, it.b, &sh.bar_q);
      tma_load_4d(q_s + kStageBytes / 2, &tm_q, 64, it.g * kHg, it.row0 + it.tile_start, it.b, &sh.bar_q);
      ++qn;
      for (int j = 0; j < it.nb; ++j) {
        ok = mbar_wait(&bar_kempty[st], ph, &give_up, 11);
        if (!ok) break;
        const uint32_t dst = k_s + st * kStageBytes;
        uint64_t* bar = &bar_kfull[st];
        mbar_arrive_expect_tx(bar, kStageBytes);
        tma_load_4d(dst, &tm_k, 0, it.g, it.row0 + j * 128, it.b, bar);
        tma_load_4d(dst + kStageBytes / 2, &tm_k, 64, it.g, it.row0 + j * 128, it.b, bar);
        if (++st == kNK) { st = 0; ph ^= 1; }
      }
    }
  };
  auto producer_tma_v = [&]() {                        // the V ring, independent of the K ring's progress
    tma_prefetch_desc(&tm_v);
    int st = 0, ph = 1;
    bool ok = true;
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      for (int j = 0; j < it.nb; ++j) {
        ok = mbar_wait(&bar_vempty[st], ph, &give_up, 12);
        if (!ok) break;
        const uint32_t dst = v_s + st * kStageBytes;
        uint64_t* bar = &bar_vfull[st];
        mbar_arrive_expect_tx(bar, kStageBytes);
        tma_load_4d(dst, &tm_v, 0, it.g, it.row0 + j * 128, it.b, bar);
        tma_load_4d(dst + kStageBytes / 2, &tm_v, 64, it.g, it.row0 + j * 128, it.b, bar);
        if (++st == kNV) { st = 0; ph ^= 1; }
      }
    }
  };

  // ================================ MMA issuer, modes without V ===================================
  // One warp issues, or (Cfg::kIssuers == 2) two, taking the key blocks in turn (global block count
  // even / odd): an issuing lane is
  // held up while the tensor core works through its queue, so with one issuer the barrier waits of
  // block n+1 would start only after block n has run; with two, one warp waits while the other's
  // products execute.  Both walk the same block sequence and keep the same counters.  A wait names a
  // barrier phase only by its parity, so an issuer must never wait on a barrier that is still two
  // phases back: the issuer of block n passes a token to the other one as soon as its own "S buffer
  // free" wait is over, and the other one starts its waits for block n+1 only then.
  auto mma_role = [&](const int me) {
    constexpr uint32_t idesc_qk = idesc_f16(128, 128, 0, 0, BF16);
    constexpr int NS = Cfg::kStreams;                   // S buffers = softmax streams; block j goes to buffer j % NS
    constexpr int kIssuers = Cfg::kIssuers;
    int k_st = 0, k_ph = 0, qn = 0, gb = 0, turns = 0;  // K ring, Q tiles, global block count, tokens taken
    int used[NS];                                      // blocks written into each S buffer so far (by either issuer)
#pragma unroll
    for (int i = 0; i < NS; ++i) used[i] = 0;
    bool ok = true;
    // the whole warp runs this role with uniform control flow; one elected lane issues
    const bool el = elect_one();
    const uint32_t q_lo = desc_lo(q_s, 16), k_lo0 = desc_lo(k_s, 16);
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      if (it.nb == 0) continue;
      ok = mbar_wait(&sh.bar_q, qn & 1, &give_up, 21);
      if (!ok) break;
      ++qn;
      int w = 0;
      bool issued_here = false;
      for (int j = 0; j < it.nb && ok; ++j, ++gb) {
        if (kIssuers == 1 || (gb & 1) == me) {
          if (kIssuers == 2 && gb > 0) {                 // the other issuer is past its waits for block gb - 1
            ok = mbar_wait(&sh.bar_turn[me], turns & 1, &give_up, 27);
            if (!ok) break;
            ++turns;
          }
          // S buffer w may be overwritten once the block issued into it before has been consumed
#pragma unroll
          for (int i = 0; i < NS; ++i) {
            if (i == w && used[i] > 0) ok = mbar_wait(&bar_pready[i], (used[i] - 1) & 1, &give_up, 23);
          }
          if (!ok) break;
          if (kIssuers == 2 && el) mbar_arrive(&sh.bar_turn[me ^ 1]);
          ok = mbar_wait(&bar_kfull[k_st], k_ph, &give_up, 22);
          if (!ok) break;
          tc_fence_after();
          const uint32_t k_lo = k_lo0 + k_st * (kStageBytes >> 4);
          const uint32_t d = t_s0 + w * 128;
          if (el) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint32_t off = (ks >> 2) * (kStageBytes / 2 / 16) + (ks & 3) * 2;
              if (POOL) mma_ss_lo(d, k_lo + off, q_lo + off, idesc_qk, ks > 0);     // S^T: lanes = keys
              else mma_ss_lo(d, q_lo + off, k_lo + off, idesc_qk, ks > 0);          // S: lanes = (query, head) rows
            }
            mma_commit(&bar_kempty[k_st]);
            mma_commit(&bar_sfull[w]);
          }
          __syncwarp();
          issued_here = true;
        }
#pragma unroll
        for (int i = 0; i < NS; ++i) if (i == w) ++used[i];
        if (++k_st == kNK) { k_st = 0; k_ph ^= 1; }
        if (++w == NS) w = 0;
      }
      if (!ok) break;
      // Q may be replaced once BOTH issuers' products of this tile have completed (two arrivals)
      if (el) {
        if (issued_here) mma_commit(&sh.bar_qempty); else mbar_arrive(&sh.bar_qempty);
      }
      __syncwarp();
    }
  };

  // ================================ MMA issuers, modes with V ======================================
  // Tensor-memory columns with V: S0, S1 (fp32, 2 x 128) | P0, P1 (fp16 pairs, 2 x 64) | O (fp32, 128).
  // Even key blocks of a tile go through (S0, P0), odd ones through (S1, P1); there is ONE accumulator.
  //
  // Two warps issue: one the Q.K^T products, one the P.V products.  An issuing lane is held up while
  // the tensor core works through what it was given, so a single issuer would spend its barrier
  // waits with the tensor core idle; with two, each warp waits while the other's products run.
  // Products of different warps are not ordered; every dependency between them goes through a
  // barrier (S consumed -> next Q.K^T into that buffer; P written -> P.V; P.V done -> P rewritten).
  auto mma_qk_v = [&]() {
    constexpr uint32_t idesc_qk = idesc_f16(128, 128, 0, 0, BF16);
    constexpr uint32_t kStage16 = kStageBytes >> 4;      // descriptor address units are 16 bytes
    const uint32_t q_lo = desc_lo(q_s, 16), k_lo0 = desc_lo(k_s, 16);
    int k_st = 0, k_ph = 0, qn = 0;                      // K ring position / parity, Q tiles seen
    int iss0 = 0, iss1 = 0;                              // blocks issued into S0 / S1 so far
    bool ok = true;
    // The whole warp runs this role with uniform control flow and one elected lane issues: addresses,
    // descriptors and ring positions are then warp-uniform values, which is what lets the tensor
    // core be fed at its own rate (a single diverged lane computing them per instruction cannot).
    const bool el = elect_one();
    if (GATHER && el) tma_prefetch_desc(&tm_q);
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      if (it.nb == 0) continue;
      if (GATHER) {
        // Sparse mode: this warp also fetches the Q tile (two TMA boxes), as soon as the previous tile's
        // last Q.K^T has completed; the next tile's Q is pulled into L2 meanwhile, so that its copy
        // starts from there.
        ok = mbar_wait(&sh.bar_qempty, (qn & 1) ^ 1, &give_up, 13);
        if (!ok) break;
        if (el) {
          mbar_arrive_expect_tx(&sh.bar_q, kStageBytes);
          tma_load_4d(q_s, &tm_q, 0, it.g * kHg, it.row0 + it.tile_start, it.b, &sh.bar_q);
          tma_load_4d(q_s + kStageBytes / 2, &tm_q, 64, it.g * kHg, it.row0 + it.tile_start, it.b, &sh.bar_q);
          if (k + 1 < n_rounds) {
            const int nitem = item_of(k + 1);
            if (nitem < n_items) {
              const TileItem nx = decode_item<MODE>(p, nitem);
              if (nx.nb > 0) {
                tma_prefetch_4d(&tm_q, 0, nx.g * kHg, nx.row0 + nx.tile_start, nx.b);
                tma_prefetch_4d(&tm_q, 64, nx.g * kHg, nx.row0 + nx.tile_start, nx.b);
              }
            }
          }
        }
        __syncwarp();
      }
      ok = mbar_wait(&sh.bar_q, qn & 1, &give_up, 21);
      if (!ok) break;
      ++qn;
      for (int j = 0; j < it.nb; ++j) {
        const int w = j & 1;
        int& iss = w ? iss1 : iss0;
        if (iss > 0) {
          // the softmax side has the previous block of this buffer in registers
          ok = mbar_wait(&sh.bar_sfree[w], (iss - 1) & 1, &give_up, 23);
          if (!ok) break;
        }
        ok = mbar_wait(&bar_kfull[k_st], k_ph, &give_up, 22);
        if (!ok) break;
        if (GATHER) fence_proxy_async_smem();            // cp.async bytes -> visible to the tensor core
        tc_fence_after();
        const uint32_t k_lo = k_lo0 + k_st * kStage16;
        const uint32_t d = t_s0 + w * 128;
        if (el) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            constexpr uint32_t kHalf16 = kStageBytes / 2 / 16;
            const uint32_t off = (ks >> 2) * kHalf16 + (ks & 3) * 2;
            mma_ss_lo(d, q_lo + off, k_lo + off, idesc_qk, ks > 0);
          }
          mma_commit(&bar_kempty[k_st]);
          mma_commit(&bar_sfull[w]);
          if (j + 1 == it.nb) mma_commit(&sh.bar_qempty);  // the tile's last Q.K^T is queued: Q may be replaced
        }
        __syncwarp();
        ++iss;
        if (++k_st == kNK) { k_st = 0; k_ph ^= 1; }
      }
    }
  };
  auto mma_pv_v = [&]() {
    constexpr uint32_t idesc_pv = idesc_f16(128, 128, 0, 1, BF16);
    constexpr uint32_t kStage16 = kStageBytes >> 4;
    const uint32_t t_acc = tmem + 384, t_p = tmem + 256;
    const uint32_t v_lo0 = desc_lo(v_s, kStageBytes / 2);
    int v_st = 0, v_ph = 0, tiles_done = 0;
    int cons0 = 0, cons1 = 0;                            // blocks consumed from P0 / P1 so far
    bool ok = true;
    const bool el = elect_one();
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      if (it.nb == 0) continue;
      for (int j = 0; j < it.nb; ++j) {
        const int w = j & 1;
        int& cons = w ? cons1 : cons0;
        ok = mbar_wait(&bar_vfull[v_st], v_ph, &give_up, 25);
        if (!ok) break;
        if (j == 0 && tiles_done > 0) {
          // the first P.V of a new tile overwrites O: the previous tile's epilogue must have read it
          ok = mbar_wait(&sh.bar_ofree, (tiles_done - 1) & 1, &give_up, 26);
          if (!ok) break;
        }
        // P(j) is in tensor memory, and O is in the scale P(j) was computed in
        ok = mbar_wait(&bar_pready[w], cons & 1, &give_up, 24);
        if (!ok) break;
        if (GATHER) fence_proxy_async_smem();
        tc_fence_after();
        const uint32_t v_lo = v_lo0 + v_st * kStage16;
        const uint32_t a = t_p + w * 64;
        if (el) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            mma_ts_lo(t_acc, a + ks * 8, v_lo + ks * (2048 >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          mma_commit(&bar_vempty[v_st]);
          mma_commit(&bar_odone[w]);
        }
        __syncwarp();
        ++cons;
        if (++v_st == kNV) { v_st = 0; v_ph ^= 1; }
      }
      if (!ok) break;
      ++tiles_done;
    }
  };

  // Softmax with V.  Warpgroup w owns the key blocks j = w, w+2, ... of every tile: a thread holds a
  // whole S row (128 values) of its block, so nothing is exchanged inside a block, and the two
  // warpgroups are naturally out of phase (one fetches and reduces while the other's exponentials
  // keep the special-function unit busy).  S(j) is free for Q.K^T(j+2) as soon as it is in
  // registers; P goes to its own tensor-memory buffer.
  //
  // Both streams accumulate into ONE O, so every row has one reference point for its exponentials,
  // decided block by block in block order: ref(j) = ref(j-1), unless the maximum of block j exceeds
  // it by more than 2^kRescaleLog2, then ref(j) = that maximum.  The owner of block j reads ref(j-1)
  // from the other warpgroup (published right after that block's maximum was known, long before its
  // exponentials are done) and publishes ref(j).  Where ref(j) != ref(j-1), which is rare, the owner of
  // block j waits for P.V(j-1) and rescales its O row before it releases P(j).  Each thread keeps
  // its part of the row sum in the reference of its own last block; the parts meet in the epilogue.
  auto softmax_role_v = [&]() {
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane, q_local = row >> 2;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ts = t_s0 + wg * 128 + lane_sel;           // this stream's S buffer
    const uint32_t tp = tmem + 256 + wg * 64 + lane_sel;      // this stream's P buffer
    const uint32_t t_acc = tmem + 384 + lane_sel;             // the O accumulator (this thread's row)
    float* ref_mine = &sh.xchg[0][wg][row];
    const float* ref_other = &sh.xchg[0][wg ^ 1][row];
    int done_mine = 0, done_other = 0, tiles_done = 0;        // blocks finished per stream, tiles finished
    bool ok = true;
    // sparse mode: the record of a tile (two dependent global loads) is fetched one tile ahead
    TileItem it_next;
    if (GATHER) it_next = decode_item<MODE>(p, min(item_of(0), n_items - 1));
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      TileItem it;
      if (GATHER) {
        it = it_next;
        if (k + 1 < n_rounds) it_next = decode_item<MODE>(p, min(item_of(k + 1), n_items - 1));
        if (item >= n_items) continue;
      } else {
        if (item >= n_items) continue;
        it = decode_item<MODE>(p, item);
      }
      if (it.nb == 0) continue;
      const int tok = it.tile_start + q_local;
      const int off = GATHER ? it.count : it.tile_start;   // slot - off = key position inside the tile
      const int n_mine = (it.nb - wg + 1) >> 1, n_other = it.nb - n_mine;
      float m_l = -INFINITY, l_run = 0.f;               // l_run is in the scale of reference m_l
      // the exchange buffer (and O) are free once both warpgroups have finished the previous tile's epilogue
      if (tiles_done > 0) {
        ok = mbar_wait(&sh.bar_ofree, (tiles_done - 1) & 1, &give_up, 37);
        if (!ok) break;
      }
      for (int j = wg, jj = 0; j < it.nb; j += 2, ++jj) {
        ok = mbar_wait(&bar_sfull[wg], (done_mine + jj) & 1, &give_up, 31);
        if (!ok) break;
        tc_fence_after();
        // the whole S row (128 fp32) comes into registers with one round trip to tensor memory
        uint32_t sr[4][32];
#pragma unroll
        for (int part = 0; part < 4; ++part) tmem_ld32(ts + part * 32, sr[part]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&sh.bar_sfree[wg]);                   // Q.K^T(j+2) may overwrite the buffer
        const int c0 = j * 128 - off;                     // key position (inside the tile) of column 0
        if ((c0 + 127) > 0) {                             // only the last block(s) of a tile
#pragma unroll
          for (int part = 0; part < 4; ++part)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if ((c0 + part * 32 + i) > q_local) sr[part][i] = 0xFF800000u;     // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        if (GATHER) {
#pragma unroll
          for (int part = 0; part < 4; ++part) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              mx0 = max3(mx0, __uint_as_float(sr[part][i]), __uint_as_float(sr[part][i + 1]));
              mx1 = max3(mx1, __uint_as_float(sr[part][i + 2]), __uint_as_float(sr[part][i + 3]));
              mx2 = max3(mx2, __uint_as_float(sr[part][i + 4]), __uint_as_float(sr[part][i + 5]));
              mx3 = max3(mx3, __uint_as_float(sr[part][i + 6]), __uint_as_float(sr[part][i + 7]));
            }
          }
        } else {
#pragma unroll
          for (int part = 0; part < 4; ++part) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              mx0 = fmaxf(mx0, __uint_as_float(sr[part][i]));
              mx1 = fmaxf(mx1, __uint_as_float(sr[part][i + 1]));
              mx2 = fmaxf(mx2, __uint_as_float(sr[part][i + 2]));
              mx3 = fmaxf(mx3, __uint_as_float(sr[part][i + 3]));
            }
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale2;
        // ---- the row's reference for this block --------------------------------------------------
        // index (in the other stream's count) of block j-1: the other stream owns j-1, j-3, ...
        const int prev_idx = done_other + ((j - 1) >> 1);
        float ref_prev = -INFINITY;
        if (j > 0) {
          ok = mbar_wait(&sh.bar_lse[wg ^ 1], prev_idx & 1, &give_up, 34);
          if (!ok) break;
          ref_prev = *ref_other;
        }
        // Probabilities stay below 2^kRescaleLog2 (exact in fp32, harmless in fp16).  A block whose
        // rows are all masked for this thread (maximum -inf) keeps the previous reference.
        const float ref = (mx > ref_prev + kRescaleLog2) ? mx : ref_prev;
        *ref_mine = ref;
        mbar_arrive(&sh.bar_lse[wg]);
        // P.V of this stream's previous block has read the P buffer
        if (done_mine + jj > 0) {
          ok = mbar_wait(&bar_odone[wg], (done_mine + jj - 1) & 1, &give_up, 38);
          if (!ok) break;
        }
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        if (GATHER) {
          // two fp32 operations per instruction: in the sparse mode the softmax warps share their issue
          // slots with six gather warps and every instruction saved shows (-4 %); in the dense mode, which
          // runs on the power cap, the same code was 2-3 % slower than the scalar form
          uint64_t s01 = 0ull, s23 = 0ull;                  // four partial row sums, two per register pair
          const uint64_t scale_2 = pair_f(p.scale2, p.scale2), nref_2 = pair_f(-ref, -ref);
#pragma unroll
          for (int part = 0; part < 4; ++part) {           // 32 keys -> 16 packed P columns
            uint32_t pr[16];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float a0, a1, a2, a3;
              unpair_f(fma2(pair_u(sr[part][2 * i], sr[part][2 * i + 1]), scale_2, nref_2), a0, a1);
              unpair_f(fma2(pair_u(sr[part][2 * i + 2], sr[part][2 * i + 3]), scale_2, nref_2), a2, a3);
              a0 = ex2(a0); a1 = ex2(a1); a2 = ex2(a2); a3 = ex2(a3);
              s01 = add2(s01, pair_f(a0, a1));
              s23 = add2(s23, pair_f(a2, a3));
              pr[i] = pack2<BF16>(a0, a1);
              pr[i + 1] = pack2<BF16>(a2, a3);
            }
            tmem_st16(tp + part * 16, pr);                 // P columns [part*16, +16) = keys [part*32, +32)
          }
          unpair_f(s01, s0, s1);
          unpair_f(s23, s2, s3);
        } else {
#pragma unroll
          for (int part = 0; part < 4; ++part) {           // 32 keys -> 16 packed P columns
            uint32_t pr[16];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float a0 = ex2(fmaf(__uint_as_float(sr[part][2 * i]), p.scale2, -ref));
              float a1 = ex2(fmaf(__uint_as_float(sr[part][2 * i + 1]), p.scale2, -ref));
              float a2 = ex2(fmaf(__uint_as_float(sr[part][2 * i + 2]), p.scale2, -ref));
              float a3 = ex2(fmaf(__uint_as_float(sr[part][2 * i + 3]), p.scale2, -ref));
              s0 += a0; s1 += a1; s2 += a2; s3 += a3;
              pr[i] = pack2<BF16>(a0, a1);
              pr[i + 1] = pack2<BF16>(a2, a3);
            }
            tmem_st16(tp + part * 16, pr);                 // P columns [part*16, +16) = keys [part*32, +32)
          }
        }
        // this thread's part of the row sum moves to the block's reference
        const float beta = (m_l == -INFINITY) ? 0.f : ex2(m_l - ref);
        l_run = l_run * beta + ((s0 + s1) + (s2 + s3));
        m_l = ref;
        if (j > 0 && __any_sync(0xFFFFFFFFu, ref != ref_prev)) {
          // O is in the scale of ref(j-1): once P.V(j-1) has landed, bring this row to ref(j).
          // (P.V(j-3) is known complete: this thread waited for P.V(j-2) above, and they complete in order.)
          ok = mbar_wait(&bar_odone[wg ^ 1], prev_idx & 1, &give_up, 32);
          if (!ok) break;
          tc_fence_after();
          const float alpha = ex2(ref_prev - ref);         // 1 for the rows whose reference stayed
#pragma unroll 1
          for (int part = 0; part < 4; ++part) {
            uint32_t orr[32];
            tmem_ld32(t_acc + part * 32, orr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st32(t_acc + part * 32, orr);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bar_pready[wg]);
      }
      if (!ok) break;
      done_mine += n_mine;
      done_other += n_other;
      // ---- epilogue: bring the two parts of the row sum together, normalise, store ----------------
      // (xchg[0][wg] already holds this stream's last reference = m_l, unless it had no block)
      if (n_mine == 0) *ref_mine = m_l;
      sh.xchg[1][wg][row] = l_run;
      mbar_arrive(&sh.bar_x);
      ok = mbar_wait(&sh.bar_x, tiles_done & 1, &give_up, 35);
      if (!ok) break;
      const float m_o = *ref_other, l_o = sh.xchg[1][wg ^ 1][row];
      const float m_tot = fmaxf(m_l, m_o);               // the reference of the tile's last block
      const float f_mine = (m_l == -INFINITY) ? 0.f : ex2(m_l - m_tot);
      const float f_other = (m_o == -INFINITY) ? 0.f : ex2(m_o - m_tot);
      const float l_tot = l_run * f_mine + l_o * f_other;
      // the tile's last P.V (own stream first: a wait may be at most one phase behind its barrier)
      if (n_mine > 0) ok = mbar_wait(&bar_odone[wg], (done_mine - 1) & 1, &give_up, 33);
      if (ok && n_other > 0) ok = mbar_wait(&bar_odone[wg ^ 1], (done_other - 1) & 1, &give_up, 36);
      if (!ok) break;
      tc_fence_after();
      const float inv = 1.0f / l_tot;
      // this warpgroup stores output columns [wg*64, +64) of its rows
      uint4 w[8];
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t oa[32];
        tmem_ld32(t_acc + wg * 64 + part * 32, oa);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          w[part * 4 + e].x = pack2<BF16>(__uint_as_float(oa[e * 8 + 0]) * inv, __uint_as_float(oa[e * 8 + 1]) * inv);
          w[part * 4 + e].y = pack2<BF16>(__uint_as_float(oa[e * 8 + 2]) * inv, __uint_as_float(oa[e * 8 + 3]) * inv);
          w[part * 4 + e].z = pack2<BF16>(__uint_as_float(oa[e * 8 + 4]) * inv, __uint_as_float(oa[e * 8 + 5]) * inv);
          w[part * 4 + e].w = pack2<BF16>(__uint_as_float(oa[e * 8 + 6]) * inv, __uint_as_float(oa[e * 8 + 7]) * inv);
        }
      }
      // O and the exchange buffer have been read: the next tile's first P.V may overwrite the accumulator
      // while this tile's rows are still on their way out
      tc_fence_before();
      mbar_arrive(&sh.bar_ofree);
      {
        // A thread holds 128 bytes of ITS row; eight neighbouring lanes transpose their eight 16-byte
        // chunks so that every store instruction writes 128 contiguous bytes per row instead of 16 (storing
        // the rows directly, 32 different lines per instruction, made the dense pass 5 % slower).  With KV
        // heads sharded over GPUs and n_fan > 1 the rows also go straight into the peers' [B, L, H_out, D]
        // buffers (plain peer stores over NVLink: the all-gather of the outputs is then this epilogue).
#pragma unroll
        for (int bit = 1; bit < 8; bit <<= 1) {
          const bool up = (lane & bit) != 0;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (c & bit) continue;
            const uint4 send = up ? w[c] : w[c | bit];
            uint4 recv;
            recv.x = __shfl_xor_sync(0xFFFFFFFFu, send.x, bit);
            recv.y = __shfl_xor_sync(0xFFFFFFFFu, send.y, bit);
            recv.z = __shfl_xor_sync(0xFFFFFFFFu, send.z, bit);
            recv.w = __shfl_xor_sync(0xFFFFFFFFu, send.w, bit);
            if (up) w[c] = recv; else w[c | bit] = recv;
          }
        }
        // now w[j] is chunk (lane & 7) of row (row & ~7) + j
        const int row0 = row & ~7, chunk = lane & 7;
        int64_t offs[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int rj = row0 + j, tj = it.tile_start + (rj >> 2);
          offs[j] = tj < it.L ? (((int64_t)it.b * p.L + it.row0 + tj) * p.H_out + p.h_off + it.g * kHg + (rj & 3)) * kD + wg * 64 + chunk * 8
                             : -1;
        }
        if (p.mc) {
          // one store per row chunk to the multicast address: the switch replicates it to every GPU
          __half* base = p.out_fan[0];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (offs[j] >= 0) multimem_st16(base + offs[j], w[j]);
        } else {
#pragma unroll 1
          for (int f = 0; f < p.n_fan; ++f) {
            __half* base = p.out_fan[f];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (offs[j] >= 0) *reinterpret_cast<uint4*>(base + offs[j]) = w[j];
          }
        }
      }
      if (wg == 0 && p.lse2 && tok < it.L)
        p.lse2[((int64_t)it.b * p.L + tok) * p.H + it.g * kHg + (row & 3)] = m_tot + log2f(l_tot);
      ++tiles_done;
    }
  };

  // ================================ softmax statistics only (no V) ================================
  // Three warpgroups, three independent streams: warpgroup w owns the key blocks j = w, w+3, ... of
  // every tile with its own S buffer and its own running (max, sum) per row, so the tcgen05.ld / max /
  // ex2 phases of one stream overlap those of the others and nothing is exchanged per block (with two
  // streams no unit was busy more than 64 %: three warps per SM sub-partition hide each other's
  // latencies better).  The partial results of a row are merged like split-K partials in the epilogue.
  auto softmax_role = [&]() {
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane, q_local = row >> 2;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ts = t_s0 + wg * 128 + lane_sel;   // this stream's S buffer
    constexpr int NS = Cfg::kStreams;
    float* const xm = xchg3;                           // [NS][128] partial maxima
    float* const xl = xchg3 + NS * 128;                // [NS][128] partial sums
    int done_mine = 0, tiles_done = 0;                 // blocks finished by this stream, tiles finished
    bool ok = true;
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      if (it.nb == 0) continue;
      const int tok = it.tile_start + q_local;
      const int off = it.tile_start;                    // slot - off = key position inside the tile
      const int n_mine = it.nb > wg ? (it.nb - wg + NS - 1) / NS : 0;
      float m_run = -INFINITY, l_run = 0.f;             // m_run in the scaled (log2) domain
      for (int j = wg, jj = 0; j < it.nb; j += NS, ++jj) {
        ok = mbar_wait(&bar_sfull[wg], (done_mine + jj) & 1, &give_up, 31);
        if (!ok) break;
        tc_fence_after();
        const int c0 = j * 128 - off;                     // key position (inside the tile) of column 0
        const bool need_mask = (c0 + 127) > 0;            // only the last block(s) of a tile
        // the whole S row (128 fp32) comes into registers with one round trip to tensor memory
        uint32_t sr[4][32];
#pragma unroll
        for (int part = 0; part < 4; ++part) tmem_ld32(ts + part * 32, sr[part]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&bar_pready[wg]);                     // S is in registers: the buffer may be refilled
        if (need_mask) {
#pragma unroll
          for (int part = 0; part < 4; ++part)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if ((c0 + part * 32 + i) > q_local) sr[part][i] = 0xFF800000u;     // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int part = 0; part < 4; ++part) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(sr[part][i]));
            mx1 = fmaxf(mx1, __uint_as_float(sr[part][i + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(sr[part][i + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(sr[part][i + 3]));
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale2;
        // The reference point of the exponentials only moves when the row maximum has grown by more
        // than 2^kRescaleLog2 (the terms then stay below 2^kRescaleLog2, exact in fp32);
        // lse2 = m + log2(l) holds for any reference point m.
        const float m_new = (mx > m_run + kRescaleLog2) ? mx : m_run;
        const float alpha = ex2(m_run - m_new);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int part = 0; part < 4; ++part)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            s0 += ex2(fmaf(__uint_as_float(sr[part][i]), p.scale2, -m_new));
            s1 += poly_also<KB200_POLY_EXTRA_LSE>(i) ? ex2_fma(fmaf(__uint_as_float(sr[part][i + 1]), p.scale2, -m_new))
                               : ex2(fmaf(__uint_as_float(sr[part][i + 1]), p.scale2, -m_new));
            s2 += ex2(fmaf(__uint_as_float(sr[part][i + 2]), p.scale2, -m_new));
            s3 += ex2_fma(fmaf(__uint_as_float(sr[part][i + 3]), p.scale2, -m_new));
          }
        l_run = l_run * alpha + ((s0 + s1) + (s2 + s3));
        m_run = m_new;
      }
      if (!ok) break;
      done_mine += n_mine;
      // ---- epilogue: merge the two streams, store ------------------------------------------------
      // the exchange buffer is free once both warpgroups have finished the previous tile's epilogue
      if (tiles_done > 0) {
        ok = mbar_wait(&sh.bar_ofree, (tiles_done - 1) & 1, &give_up, 37);
        if (!ok) break;
      }
      xm[wg * 128 + row] = m_run;
      xl[wg * 128 + row] = l_run;
      mbar_arrive(&sh.bar_x);
      ok = mbar_wait(&sh.bar_x, tiles_done & 1, &give_up, 35);
      if (!ok) break;
      if (wg == 0 && p.lse2 && tok < it.L) {
        float m_tot = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < NS; ++s2) m_tot = fmaxf(m_tot, xm[s2 * 128 + row]);
        float l_tot = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < NS; ++s2) {
          const float ms = xm[s2 * 128 + row];
          if (ms != -INFINITY) l_tot += xl[s2 * 128 + row] * ex2(ms - m_tot);
        }
        p.lse2[((int64_t)it.b * p.L + tok) * p.H + it.g * kHg + (row & 3)] = m_tot + log2f(l_tot);
      }
      // the exchange buffer has been read
      mbar_arrive(&sh.bar_ofree);
      ++tiles_done;
    }
  };

  // ================================ pooled-score reducer =========================================
  // warpgroup w owns the key blocks j = w, w+3, ... of every tile; thread = key lane, sums over the
  // tile's 128 (query, head) rows, i.e. over the 128 columns of S^T
  auto pool_role = [&]() {
    const int wg = warp >> 2;
    const int key_lane = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ts = t_s0 + wg * 128 + lane_sel;
    int done_mine = 0, tiles_seen = 0;
    bool ok = true;
    for (int k = 0; k < n_rounds && ok; ++k) {
      const int item = item_of(k);
      if (item >= n_items) continue;
      const TileItem it = decode_item<MODE>(p, item);
      if (it.nb == 0) continue;
      constexpr int NS = Cfg::kStreams;
      const int n_mine = it.nb > wg ? (it.nb - wg + NS - 1) / NS : 0;
      // this warpgroup's copy of the tile's 128 lse2 values (row = 4 * query + head), double-buffered
      // by tile parity: a thread that runs ahead must not overwrite values that a slower thread of
      // the warpgroup still reads for the previous tile
      float* lse_s = xchg3 + (wg * 2 + (tiles_seen & 1)) * 128;
      {
        const int tok = it.tile_start + (key_lane >> 2);
        lse_s[key_lane] =
            tok < it.L ? -p.lse2_in[((int64_t)it.b * p.L + tok) * p.H + it.g * kHg + (key_lane & 3)] : -INFINITY;
        mbar_arrive(&sh.bar_lse[wg]);
        ok = mbar_wait(&sh.bar_lse[wg], tiles_seen & 1, &give_up, 43);
        if (!ok) break;
        ++tiles_seen;
      }
      float* prow = p.pooled + (((int64_t)it.b * p.G + it.g) * p.T + it.t) * p.pooled_stride;
      for (int j = wg, jj = 0; j < it.nb; j += NS, ++jj) {
        ok = mbar_wait(&bar_sfull[wg], (done_mine + jj) & 1, &give_up, 41);
        if (!ok) break;
        tc_fence_after();
        uint64_t a01 = 0ull, a23 = 0ull;                    // four partial sums, two per register pair
        const uint64_t scale_2 = pair_f(p.scale2, p.scale2);
        uint32_t sr[4][32];
#pragma unroll
        for (int part = 0; part < 4; ++part) tmem_ld32(ts + part * 32, sr[part]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&bar_pready[wg]);                      // S^T block is in registers: the buffer is free
#pragma unroll
        for (int part = 0; part < 4; ++part)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            // the four rows' lse2 with one 16-byte shared-memory load (the same address for the whole warp)
            const float4 l4 = reinterpret_cast<const float4*>(lse_s)[part * 8 + (i >> 2)];   // holds -lse2
            float x0, x1, x2, x3;
            unpair_f(fma2(pair_u(sr[part][i], sr[part][i + 1]), scale_2, pair_f(l4.x, l4.y)), x0, x1);
            unpair_f(fma2(pair_u(sr[part][i + 2], sr[part][i + 3]), scale_2, pair_f(l4.z, l4.w)), x2, x3);
            a01 = add2(a01, pair_f(ex2(x0), poly_also<KB200_POLY_EXTRA_POOL>(i) ? ex2_fma(x1) : ex2(x1)));
            a23 = add2(a23, pair_f(ex2(x2), ex2_fma(x3)));
          }
        float a0, a1, a2, a3;
        unpair_f(a01, a0, a1);
        unpair_f(a23, a2, a3);
        const int key = j * 128 + key_lane;
        if (key < it.tile_start) prow[key] = (a0 + a1) + (a2 + a3);
      }
      done_mine += n_mine;
    }
  };

  // ================================ role dispatch =================================================
  // Register hand-over (setmaxnreg).  The pool is what the CTA got at launch: the softmax warpgroups
  // can only take what the other warpgroups give back, and the warps that share an SM sub-partition
  // (w, w+4, w+8, w+12) must stay within 512 registers per thread slot.
  //   sparse: 512 threads x 128 at launch; 256 x 200 + 256 x 56 = 65536; 2 x 200 + 2 x 56 = 512
  //   dense : 384 threads x 168 at launch; 256 x 200 + 128 x 96 = 63488 <= 64512; 2 x 200 + 96 <= 512
  // The instruction is warpgroup-wide: all four warps of a warpgroup execute the same one, and the role
  // code sits inside the branch that issued it.
  if (!HAS_V) {
    //   no V : 512 threads x 128 at launch; 384 x 152 + 128 x 56 = 65536; 3 x 152 + 56 = 512
    if (warp < Cfg::kSoftmaxWarps) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 152;\n");
      if (POOL) pool_role(); else softmax_role();
    } else {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n");
      if (warp == Cfg::kProducerWarp0) {
        if (lane == 0) producer_tma();
        __syncwarp();
      } else if (warp == kMmaWarp) {
        mma_role(0);
      } else if (Cfg::kIssuers == 2 && warp == kMmaWarp + 1) {
        mma_role(1);
      }
    }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;\n");
    softmax_role_v();
  } else if (GATHER) {
    if (warp < 12) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n");
      producer_gather();
    } else {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n");
      if (warp == kMmaWarp) mma_qk_v();
      else if (warp == kMmaWarp + 1) mma_pv_v();
      else producer_gather();
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;\n");
    if (warp == Cfg::kProducerWarp0) {
      if (lane == 0) producer_tma();
      __syncwarp();
    } else if (warp == kMmaWarp) {
      mma_qk_v();
    } else if (warp == kMmaWarp + 1) {
      if (lane == 0) producer_tma_v();
      __syncwarp();
    } else if (warp == kMmaWarp + 2) {
      mma_pv_v();
    }
  }

  // ---- teardown: every role ends up here, also after a wait that gave up ----------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
  if (tid == 0 && give_up != 0) atomicCAS(&g_status_word, 0, give_up);
}

// The give-up path of the bounded waits, exercised on purpose and harmlessly: one CTA allocates tensor
// memory like the prefill kernels, then every thread waits (with a limit of `limit_ns`) on a barrier on
// which nobody ever arrives.  The wait must run out, the first thread to notice records `code`, the others
// see the flag and leave too, the CTA frees its tensor memory, publishes the code in the device status
// word (the one kb200_read_status returns and clears) and returns.  result[0] = the code the CTA ended
// with, result[1] = number of threads whose wait returned false, result[2] = elapsed nanoseconds.
__global__ void __launch_bounds__(128, 1)
selftest_wait_timeout_kernel(int32_t* __restrict__ result, unsigned long long limit_ns, int code) {
  using namespace umma;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int give_up;
  __shared__ int n_false;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    give_up = 0;
    n_false = 0;
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_sh, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint64_t t0 = global_ns();
  const bool ok = mbar_wait_limit(&bar, 0, &give_up, code, limit_ns);   // nobody arrives: must return false
  if (!ok) atomicAdd(&n_false, 1);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base_sh, 32);
  if (tid == 0) {
    if (give_up != 0) atomicCAS(&g_status_word, 0, give_up);
    result[0] = give_up;
    result[1] = n_false;
    result[2] = (int32_t)min((unsigned long long)(global_ns() - t0), 0x7FFFFFFFull);
  }
}

// ---- host side ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;

int init_prefill() {
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kDenseAttn, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kSparse, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kDenseLse, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemNoV));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kPool, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemNoV));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kDenseAttn, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kSparse, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kDenseLse, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemNoV));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kPool, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemNoV));
  if (!g_encode_tiled) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult res;
    KB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &res));
    KB_REQUIRE(res == cudaDriverEntryPointSuccess && fn, "the driver does not export cuTensorMapEncodeTiled");
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  }
  return 0;
}

// 4-D tiled map over fp16 activations: dimensions (d, head, token, batch), 128-byte swizzle, boxes of
// 64 x box_heads x box_tokens x 1 elements.  Host-only work (the descriptor is passed by value).
// Encoded descriptors are kept in a small table keyed by (pointer, strides, extents, box): a serving
// loop presents the same few layouts again and again (one per layer buffer), so steady-state calls
// encode nothing.  A descriptor holds no device state, so an entry never goes stale: the same key
// always encodes to the same bytes.
struct MapKey {
  const void* base;
  int64_t sb, st, sh;
  int heads, tokens, batch, box_heads, box_tokens;
  bool operator==(const MapKey& o) const {
    return base == o.base && sb == o.sb && st == o.st && sh == o.sh && heads == o.heads && tokens == o.tokens &&
           batch == o.batch && box_heads == o.box_heads && box_tokens == o.box_tokens;
  }
};
constexpr int kMapCacheSize = 128;
static MapKey g_map_keys[kMapCacheSize];
static CUtensorMap g_map_vals[kMapCacheSize];
static int g_map_used = 0, g_map_next = 0;
static std::mutex g_map_mutex;
static std::atomic<long long> g_map_encodes{0};

static int make_act_map(CUtensorMap* map, const __half* base, int64_t sb, int64_t st, int64_t sh, int heads,
                        int tokens, int batch, int box_heads, int box_tokens, const char* what) {
  KB_REQUIRE(g_encode_tiled, "kb200_init has not been called");
  // a dimension of extent 1 never uses its stride; give it a legal one
  const int64_t min_stride = 8;
  if (heads == 1 && sh < min_stride) sh = kD;
  if (batch == 1 && sb < min_stride) sb = (int64_t)tokens * (st > 0 ? st : kD);
  const MapKey key{base, sb, st, sh, heads, tokens, batch, box_heads, box_tokens};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    for (int i = 0; i < g_map_used; ++i)
      if (g_map_keys[i] == key) {
        *map = g_map_vals[i];
        return 0;
      }
  }
  const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)heads, (cuuint64_t)tokens, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2, (cuuint64_t)sb * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_tokens, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<__half*>(base), dims, strides, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  KB_REQUIRE(r == CUDA_SUCCESS,
             "prefill: cuTensorMapEncodeTiled rejected the layout of %s (error %d; strides b/t/h = %lld/%lld/%lld)", what,
             (int)r, (long long)sb, (long long)st, (long long)sh);
  g_map_encodes.fetch_add(1);
  std::lock_guard<std::mutex> lock(g_map_mutex);
  const int slot = g_map_used < kMapCacheSize ? g_map_used++ : (g_map_next++ % kMapCacheSize);
  g_map_keys[slot] = key;
  g_map_vals[slot] = *map;
  return 0;
}

static int fill_act(const kb200_act_layout* a, const __half** ptr, int64_t* sb, int64_t* st, int64_t* sh,
                    const char* what) {
  KB_REQUIRE(a && a->ptr, "prefill: %s is null", what);
  KB_REQUIRE((reinterpret_cast<uintptr_t>(a->ptr) & 15) == 0 && a->stride_b % 8 == 0 && a->stride_t % 8 == 0 &&
                 a->stride_h % 8 == 0,
             "prefill: %s must be 16-byte aligned with strides that are multiples of 8 elements", what);
  KB_REQUIRE(a->dtype == KB200_FP16 || a->dtype == KB200_BF16, "prefill: %s has an unknown dtype code %d", what, a->dtype);
  *ptr = static_cast<const __half*>(a->ptr);
  *sb = a->stride_b;
  *st = a->stride_t;
  *sh = a->stride_h;
  return 0;
}

// Where the output rows go: one buffer of this call's heads, or (fan != NULL) the same rows into
// several [B, L, total_heads, D] buffers at head_offset.
static int set_outputs(PrefillParams* p, void* out, const kb200_out_fanout* fan, int num_q_heads, const char* what) {
  if (!fan) {
    KB_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0, "%s: out must be 16-byte aligned", what);
    p->out = static_cast<__half*>(out);
    p->out_fan[0] = p->out;
    p->n_fan = 1;
    p->H_out = num_q_heads;
    p->h_off = 0;
    p->mc = 0;
    return 0;
  }
  KB_REQUIRE(fan->count >= 1 && fan->count <= KB200_MAX_FANOUT, "%s: fan-out of %d outputs (1..%d supported)", what,
             fan->count, KB200_MAX_FANOUT);
  KB_REQUIRE(fan->head_offset >= 0 && fan->total_heads >= num_q_heads &&
                 fan->head_offset <= fan->total_heads - num_q_heads,
             "%s: heads [%d, %d) do not fit an output row of %d heads", what, fan->head_offset,
             fan->head_offset + num_q_heads, fan->total_heads);
  for (int i = 0; i < fan->count; ++i) {
    KB_REQUIRE(fan->out[i] && (reinterpret_cast<uintptr_t>(fan->out[i]) & 15) == 0,
               "%s: fan-out output %d is null or not 16-byte aligned", what, i);
    p->out_fan[i] = static_cast<__half*>(fan->out[i]);
  }
  KB_REQUIRE(fan->multicast == 0 || (fan->multicast == 1 && fan->count == 1),
             "%s: a multicast fan-out takes exactly one (multicast) address", what);
  p->mc = fan->multicast;
  p->out = p->out_fan[0];
  p->n_fan = fan->count;
  p->H_out = fan->total_heads;
  p->h_off = fan->head_offset;
  return 0;
}

// How many (sequence, KV head) pairs to walk together: as many as keep their K (and V) within about
// half of the 126 MB L2, at least one, a divisor of B * G.
static int pick_group(int batch, int groups, int seq_len, bool with_v) {
  const int64_t per_pair = (int64_t)seq_len * kD * 2 * (with_v ? 2 : 1);
  const int nbg = batch * groups;
  int want = (int)std::max<int64_t>(1, std::min<int64_t>(nbg, (64ll << 20) / std::max<int64_t>(per_pair, 1)));
  while (nbg % want != 0) --want;
  return want;
}

// one CTA per SM (the kernels are persistent), fewer when there are fewer tiles than SMs
static unsigned persistent_grid(const PrefillParams& p) {
  int64_t items = (int64_t)p.B * p.G * p.T;
  int64_t sms = sm_count();
  return (unsigned)(items < sms ? items : sms);
}

static int check_shape(const kb200_act_layout* q, int batch, int seq_len, int H, int G) {
  KB_ENTRY(q ? q->ptr : nullptr, "prefill: q");
  KB_REQUIRE(batch >= 0 && seq_len >= 0, "prefill: negative size");
  KB_REQUIRE(G > 0 && H == G * kHg,
             "prefill: %d query heads / %d KV heads; exactly %d query heads per KV head are supported", H, G, kHg);
  KB_REQUIRE((int64_t)batch * G * ceil_div(seq_len > 0 ? seq_len : 1, kTile) < (1ll << 30), "prefill: too many tiles");
  return 0;
}

}  // namespace kb200

extern "C" long long kb200_tensor_map_encodes(void) { return kb200::g_map_encodes.load(); }

extern "C" int kb200_read_status(int* host_out) {
  using namespace kb200;
  KB_REQUIRE(host_out, "read_status: null pointer");
  int zero = 0;
  KB_CUDA(cudaMemcpyFromSymbol(host_out, g_status_word, sizeof(int)));
  KB_CUDA(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
  return 0;
}

extern "C" int kb200_selftest_wait_timeout(int32_t* result, uint64_t limit_ns, int code, void* stream) {
  using namespace kb200;
  KB_ENTRY(result, "selftest_wait_timeout: result");
  KB_REQUIRE(result, "selftest_wait_timeout: null pointer");
  KB_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ull, "selftest_wait_timeout: limit must lie in (0, 100 ms]");
  KB_REQUIRE(code > 0 && code < 256, "selftest_wait_timeout: code must lie in [1, 255]");
  selftest_wait_timeout_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(result, (unsigned long long)limit_ns, code);
  KB_CHECK_LAUNCH("selftest_wait_timeout_kernel");
  return 0;
}

namespace kb200 {
// q, k (and v) must share one storage type; the outputs are written in it
static int same_dtype(PrefillParams* p, const kb200_act_layout* q, const kb200_act_layout* k, const kb200_act_layout* v,
                      const char* what) {
  KB_REQUIRE(q->dtype == k->dtype && (!v || !v->ptr || v->dtype == q->dtype),
             "%s: q, k and v must have the same dtype (codes %d / %d / %d)", what, q->dtype, k->dtype, v ? v->dtype : -1);
  p->bf16 = q->dtype == KB200_BF16;
  return 0;
}

static int set_ragged(PrefillParams* p, const kb200_ragged* rg, const char* what) {
  p->seq_start = nullptr;
  p->seq_len = nullptr;
  if (!rg) return 0;
  KB_REQUIRE(rg->seq_len, "%s: a ragged batch needs seq_len", what);
  p->seq_start = rg->seq_start;
  p->seq_len = rg->seq_len;
  return 0;
}

static int prefill_dense_impl(const kb200_act_layout* q, const kb200_act_layout* k, const kb200_act_layout* v,
                              float softmax_scale, void* out, const kb200_out_fanout* fan, float* lse2, int batch,
                              int seq_len, int num_q_heads, int num_kv_heads, void* stream,
                              const kb200_ragged* rg = nullptr) {
  if (check_shape(q, batch, seq_len, num_q_heads, num_kv_heads) != 0) return -1;
  if (fan) out = fan->count >= 1 ? fan->out[0] : nullptr;
  KB_REQUIRE(out || lse2, "prefill_dense: nothing to compute (out and lse2 are both null)");
  if (batch == 0 || seq_len == 0) return 0;
  PrefillParams p{};
  if (fill_act(q, &p.q, &p.q_sb, &p.q_st, &p.q_sh, "q") != 0) return -1;
  if (fill_act(k, &p.k, &p.k_sb, &p.k_st, &p.k_sh, "k") != 0) return -1;
  if (out && fill_act(v, &p.v, &p.v_sb, &p.v_st, &p.v_sh, "v") != 0) return -1;
  if (out && set_outputs(&p, out, fan, num_q_heads, "prefill_dense") != 0) return -1;
  p.scale2 = softmax_scale * kLog2e;
  p.lse2 = lse2;
  p.B = batch; p.L = seq_len; p.H = num_q_heads; p.G = num_kv_heads; p.T = ceil_div(seq_len, kTile);
  if (set_ragged(&p, rg, "prefill_dense") != 0) return -1;
  p.group = pick_group(batch, num_kv_heads, seq_len, out != nullptr);
  CUtensorMap tq, tk, tv;
  if (make_act_map(&tq, p.q, p.q_sb, p.q_st, p.q_sh, num_q_heads, seq_len, batch, kHg, kTile, "q") != 0) return -1;
  if (make_act_map(&tk, p.k, p.k_sb, p.k_st, p.k_sh, num_kv_heads, seq_len, batch, 1, 128, "k") != 0) return -1;
  tv = tk;
  if (out && make_act_map(&tv, p.v, p.v_sb, p.v_st, p.v_sh, num_kv_heads, seq_len, batch, 1, 128, "v") != 0) return -1;
  dim3 grid(persistent_grid(p));
  if (same_dtype(&p, q, k, out ? v : nullptr, "prefill_dense") != 0) return -1;
  if (out && p.bf16)
    tile_prefill_kernel<kDenseAttn, true><<<grid, PfCfg<kDenseAttn>::kThreads, kSmemAttn, (cudaStream_t)stream>>>(p, tq, tk, tv);
  else if (out)
    tile_prefill_kernel<kDenseAttn, false><<<grid, PfCfg<kDenseAttn>::kThreads, kSmemAttn, (cudaStream_t)stream>>>(p, tq, tk, tv);
  else if (p.bf16)
    tile_prefill_kernel<kDenseLse, true><<<grid, PfCfg<kDenseLse>::kThreads, kSmemNoV, (cudaStream_t)stream>>>(p, tq, tk, tv);
  else
    tile_prefill_kernel<kDenseLse, false><<<grid, PfCfg<kDenseLse>::kThreads, kSmemNoV, (cudaStream_t)stream>>>(p, tq, tk, tv);
  KB_CHECK_LAUNCH("tile_prefill_kernel<dense>");
  return 0;
}
}  // namespace kb200

extern "C" int kb200_prefill_dense(const kb200_act_layout* q, const kb200_act_layout* k,
                                   const kb200_act_layout* v, float softmax_scale, void* out, float* lse2,
                                   int batch, int seq_len, int num_q_heads, int num_kv_heads, void* stream) {
  return kb200::prefill_dense_impl(q, k, v, softmax_scale, out, nullptr, lse2, batch, seq_len, num_q_heads,
                                   num_kv_heads, stream);
}

extern "C" int kb200_prefill_dense_fanout(const kb200_act_layout* q, const kb200_act_layout* k,
                                          const kb200_act_layout* v, float softmax_scale,
                                          const kb200_out_fanout* fan, float* lse2, int batch, int seq_len,
                                          int num_q_heads, int num_kv_heads, void* stream) {
  using namespace kb200;
  KB_REQUIRE(fan, "prefill_dense_fanout: fan is null");
  return prefill_dense_impl(q, k, v, softmax_scale, nullptr, fan, lse2, batch, seq_len, num_q_heads, num_kv_heads,
                            stream);
}

namespace kb200 {
static int prefill_pool_impl(const kb200_act_layout* q, const kb200_act_layout* k, const float* lse2,
                             float softmax_scale, float* pooled, int64_t row_stride, int batch, int seq_len,
                             int num_q_heads, int num_kv_heads, void* stream, const kb200_ragged* rg) {
  if (check_shape(q, batch, seq_len, num_q_heads, num_kv_heads) != 0) return -1;
  KB_REQUIRE(lse2 && pooled, "prefill_pool_scores: null pointer");
  KB_REQUIRE(row_stride >= seq_len, "prefill_pool_scores: row_stride (%lld) smaller than seq_len (%d)",
             (long long)row_stride, seq_len);
  if (batch == 0 || seq_len == 0) return 0;
  PrefillParams p{};
  if (fill_act(q, &p.q, &p.q_sb, &p.q_st, &p.q_sh, "q") != 0) return -1;
  if (fill_act(k, &p.k, &p.k_sb, &p.k_st, &p.k_sh, "k") != 0) return -1;
  p.scale2 = softmax_scale * kLog2e;
  p.lse2_in = lse2;
  p.pooled = pooled;
  p.pooled_stride = row_stride;
  p.B = batch; p.L = seq_len; p.H = num_q_heads; p.G = num_kv_heads; p.T = ceil_div(seq_len, kTile);
  if (set_ragged(&p, rg, "prefill_pool_scores") != 0) return -1;
  p.group = pick_group(batch, num_kv_heads, seq_len, false);
  CUtensorMap tq, tk;
  if (make_act_map(&tq, p.q, p.q_sb, p.q_st, p.q_sh, num_q_heads, seq_len, batch, kHg, kTile, "q") != 0) return -1;
  if (make_act_map(&tk, p.k, p.k_sb, p.k_st, p.k_sh, num_kv_heads, seq_len, batch, 1, 128, "k") != 0) return -1;
  dim3 grid(persistent_grid(p));
  if (same_dtype(&p, q, k, nullptr, "prefill_pool_scores") != 0) return -1;
  if (p.bf16)
    tile_prefill_kernel<kPool, true><<<grid, PfCfg<kPool>::kThreads, kSmemNoV, (cudaStream_t)stream>>>(p, tq, tk, tk);
  else
    tile_prefill_kernel<kPool, false><<<grid, PfCfg<kPool>::kThreads, kSmemNoV, (cudaStream_t)stream>>>(p, tq, tk, tk);
  KB_CHECK_LAUNCH("tile_prefill_kernel<pool>");
  return 0;
}
}  // namespace kb200

extern "C" int kb200_prefill_pool_scores(const kb200_act_layout* q, const kb200_act_layout* k,
                                         const float* lse2, float softmax_scale, float* pooled,
                                         int64_t row_stride, int batch, int seq_len, int num_q_heads,
                                         int num_kv_heads, void* stream) {
  return kb200::prefill_pool_impl(q, k, lse2, softmax_scale, pooled, row_stride, batch, seq_len, num_q_heads,
                                  num_kv_heads, stream, nullptr);
}

extern "C" int kb200_prefill_pool_scores_ragged(const kb200_act_layout* q, const kb200_act_layout* k,
                                                const float* lse2, float softmax_scale, float* pooled,
                                                int64_t row_stride, const kb200_ragged* ragged, int batch, int max_len,
                                                int num_q_heads, int num_kv_heads, void* stream) {
  using namespace kb200;
  KB_REQUIRE(ragged, "prefill_pool_scores_ragged: ragged is null");
  return prefill_pool_impl(q, k, lse2, softmax_scale, pooled, row_stride, batch, max_len, num_q_heads, num_kv_heads,
                           stream, ragged);
}

extern "C" int kb200_prefill_dense_ragged(const kb200_act_layout* q, const kb200_act_layout* k,
                                          const kb200_act_layout* v, float softmax_scale, void* out, float* lse2,
                                          const kb200_ragged* ragged, int batch, int max_len, int num_q_heads,
                                          int num_kv_heads, void* stream) {
  using namespace kb200;
  KB_REQUIRE(ragged, "prefill_dense_ragged: ragged is null");
  return prefill_dense_impl(q, k, v, softmax_scale, out, nullptr, lse2, batch, max_len, num_q_heads, num_kv_heads,
                            stream, ragged);
}

namespace kb200 {
static int prefill_sparse_impl(const kb200_act_layout* q, const kb200_act_layout* k, const kb200_act_layout* v,
                               const int32_t* tile_idx, int64_t idx_stride, const int32_t* tile_count,
                               const int32_t* head_map, float softmax_scale, void* out, const kb200_out_fanout* fan,
                               float* lse2, int batch, int seq_len, int num_q_heads, int num_kv_heads,
                               int idx_kv_heads, void* stream, const kb200_ragged* rg = nullptr) {
  if (check_shape(q, batch, seq_len, num_q_heads, num_kv_heads) != 0) return -1;
  if (fan) out = fan->count >= 1 ? fan->out[0] : nullptr;
  KB_REQUIRE(tile_idx && tile_count && out, "prefill_sparse: null pointer");
  KB_REQUIRE(idx_stride >= 0, "prefill_sparse: negative idx_stride");
  KB_REQUIRE(idx_kv_heads == 0 || head_map || idx_kv_heads == num_kv_heads,
             "prefill_sparse: idx_kv_heads differs from num_kv_heads, so a head_map is required");
  if (batch == 0 || seq_len == 0) return 0;
  PrefillParams p{};
  if (fill_act(q, &p.q, &p.q_sb, &p.q_st, &p.q_sh, "q") != 0) return -1;
  if (fill_act(k, &p.k, &p.k_sb, &p.k_st, &p.k_sh, "k") != 0) return -1;
  if (fill_act(v, &p.v, &p.v_sb, &p.v_st, &p.v_sh, "v") != 0) return -1;
  // the gather computes row addresses as key * (token stride in bytes) with a 32-bit factor
  KB_REQUIRE(p.k_st >= 0 && p.k_st < (1ll << 29) && p.v_st >= 0 && p.v_st < (1ll << 29),
             "prefill_sparse: token strides of k and v must lie in [0, 2^29) elements");
  p.tile_idx = tile_idx;
  p.G_idx = idx_kv_heads > 0 ? idx_kv_heads : num_kv_heads;
  p.idx_stride = idx_stride;
  p.tile_count = tile_count;
  p.head_map = head_map;
  p.scale2 = softmax_scale * kLog2e;
  if (set_outputs(&p, out, fan, num_q_heads, "prefill_sparse") != 0) return -1;
  p.lse2 = lse2;
  p.B = batch; p.L = seq_len; p.H = num_q_heads; p.G = num_kv_heads; p.T = ceil_div(seq_len, kTile);
  if (set_ragged(&p, rg, "prefill_sparse") != 0) return -1;
  p.group = pick_group(batch, num_kv_heads, seq_len, true);
  CUtensorMap tq, none{};                                // Q tiles by TMA; the K / V rows are gathered without maps
  if (make_act_map(&tq, p.q, p.q_sb, p.q_st, p.q_sh, num_q_heads, seq_len, batch, kHg, kTile, "q") != 0) return -1;
  dim3 grid(persistent_grid(p));
  if (same_dtype(&p, q, k, v, "prefill_sparse") != 0) return -1;
  if (p.bf16)
    tile_prefill_kernel<kSparse, true><<<grid, PfCfg<kSparse>::kThreads, kSmemAttn, (cudaStream_t)stream>>>(p, tq, none, none);
  else
    tile_prefill_kernel<kSparse, false><<<grid, PfCfg<kSparse>::kThreads, kSmemAttn, (cudaStream_t)stream>>>(p, tq, none, none);
  KB_CHECK_LAUNCH("tile_prefill_kernel<sparse>");
  return 0;
}
}  // namespace kb200

extern "C" int kb200_prefill_sparse(const kb200_act_layout* q, const kb200_act_layout* k,
                                    const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                                    const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                                    void* out, float* lse2, int batch, int seq_len, int num_q_heads,
                                    int num_kv_heads, int idx_kv_heads, void* stream) {
  return kb200::prefill_sparse_impl(q, k, v, tile_idx, idx_stride, tile_count, head_map, softmax_scale, out, nullptr,
                                    lse2, batch, seq_len, num_q_heads, num_kv_heads, idx_kv_heads, stream);
}

extern "C" int kb200_prefill_sparse_fanout(const kb200_act_layout* q, const kb200_act_layout* k,
                                           const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                                           const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                                           const kb200_out_fanout* fan, float* lse2, int batch, int seq_len,
                                           int num_q_heads, int num_kv_heads, int idx_kv_heads, void* stream) {
  using namespace kb200;
  KB_REQUIRE(fan, "prefill_sparse_fanout: fan is null");
  return prefill_sparse_impl(q, k, v, tile_idx, idx_stride, tile_count, head_map, softmax_scale, nullptr, fan, lse2,
                             batch, seq_len, num_q_heads, num_kv_heads, idx_kv_heads, stream);
}

extern "C" int kb200_prefill_sparse_ragged(const kb200_act_layout* q, const kb200_act_layout* k,
                                           const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                                           const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                                           void* out, float* lse2, const kb200_ragged* ragged, int batch, int max_len,
                                           int num_q_heads, int num_kv_heads, int idx_kv_heads, void* stream) {
  using namespace kb200;
  KB_REQUIRE(ragged, "prefill_sparse_ragged: ragged is null");
  return prefill_sparse_impl(q, k, v, tile_idx, idx_stride, tile_count, head_map, softmax_scale, out, nullptr, lse2,
                             batch, max_len, num_q_heads, num_kv_heads, idx_kv_heads, stream, ragged);
}
