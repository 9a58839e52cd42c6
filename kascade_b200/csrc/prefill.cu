// Tile prefill kernels on the sm_100a tensor-core path (tcgen05.mma, accumulators in tensor memory).
//
// One CTA owns one query tile: 32 consecutive queries x the 4 query heads of one KV head = 128
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
// Warp roles (416 threads): warps 0-7 softmax / reducer — two warpgroups, each thread owns one
// tensor-memory lane and one half of the 128 columns of a block, so that two warps per SM
// sub-partition overlap their tcgen05.ld / ex2 / FMA chains; warps 8-11 producers (cp.async 16-byte
// chunks, 16 lanes per 256-byte row, written in the 128-byte-swizzled operand layout of umma.cuh);
// warp 12 issues the MMAs from one thread (warps 13-15 complete its warpgroup and idle, so that
// setmaxnreg can move registers from the producer / MMA warpgroups to the softmax warpgroups).
// Hand-offs are mbarriers; every wait is bounded (umma::mbar_wait) and a kernel that gives up
// records a code in the device status word, drains its copies, frees its tensor memory and returns.
//
// Tensor memory (512 columns): S0 [0,128), S1 [128,256), O0 [256,384), O1 [384,512): key blocks of even
// and odd index form two independent streams (own S buffer, own O accumulator, own softmax warpgroup).
// P (fp16) overwrites the first 64 columns of the S buffer it was computed from and is the A operand
// of the P.V product.
#include "common.cuh"
#include "umma.cuh"

namespace kb200 {

enum PrefillMode { kDenseAttn = 0, kDenseLse = 1, kSparse = 2, kPool = 3 };

constexpr int kSoftmaxThreads = 256;             // warps 0-7
constexpr int kProducerWarp0 = 8;                // warps 8-11
constexpr int kMmaWarp = 12;
constexpr int kPfThreads = 16 * 32;               // warps 13-15 only pad the last warpgroup
constexpr int kStageBytes = 128 * kD * 2;     // one 128-row operand tile (32 KB)
constexpr int kNKMax = 6;                     // K ring: 3 stages with a V ring, 6 without
constexpr int kNV = 3;

__device__ int g_status_word = 0;

struct PrefillParams {
  const __half* q; int64_t q_sb, q_st, q_sh;
  const __half* k; int64_t k_sb, k_st, k_sh;
  const __half* v; int64_t v_sb, v_st, v_sh;
  const int32_t* tile_idx; int64_t idx_stride;
  const int32_t* tile_count;
  const int32_t* head_map;
  float scale2;
  __half* out;
  float* lse2;
  const float* lse2_in;
  float* pooled; int64_t pooled_stride;
  int B, L, H, G, T;
  int G_idx;                      // KV heads in the index tensors (>= G when heads are sharded)
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
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Barriers and small exchange buffers; lives in dynamic shared memory behind the operand tiles so that
// the 7 x 32 KB tiles, the alignment padding and this block together stay inside the 227 KB limit.
struct PfShared {
  uint64_t bar_q, bar_kfull[kNKMax], bar_kempty[kNKMax], bar_vfull[kNV], bar_vempty[kNV];
  uint64_t bar_sfull[2], bar_pready[2], bar_odone[2], bar_x;
  uint32_t tmem;
  int give_up;
  float xchg[2][2][128];                               // [block parity][column half][row]
};
constexpr float kRescaleLog2 = 8.0f;                   // see the softmax role
constexpr int kPadAllowance = 768;                     // tiles need 1024-byte alignment

template <int MODE>
__global__ void __launch_bounds__(kPfThreads, 1) tile_prefill_kernel(const PrefillParams p) {
  using namespace umma;
  constexpr bool HAS_V = MODE == kDenseAttn || MODE == kSparse;
  constexpr bool POOL = MODE == kPool;
  constexpr bool GATHER = MODE == kSparse;
  constexpr int kNK = HAS_V ? 3 : kNKMax;             // K ring depth

  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = (int)gridDim.x - 1 - (int)blockIdx.x;   // long tiles first
  const int g = blockIdx.y, b = blockIdx.z;
  const int tile_start = t * kTile;
  const int rows_valid = min(kTile, p.L - tile_start);

  int count = 0, total;
  const int32_t* idx_row = nullptr;
  if (GATHER) {
    const int src_g = p.head_map ? p.head_map[g] : g;
    const int64_t r = ((int64_t)b * p.G_idx + src_g) * p.T + t;
    count = p.tile_count[r];
    count = max(0, min(count, (int)min((int64_t)tile_start, p.idx_stride)));
    idx_row = p.tile_idx + r * p.idx_stride;
    total = count + rows_valid;
  } else if (POOL) {
    total = tile_start;
  } else {
    total = tile_start + rows_valid;
  }
  const int nb = (total + 127) >> 7;
  if (nb == 0) return;                                   // pool pass of tile 0: no earlier keys
  // an earlier CTA or kernel gave up a bounded wait: do not queue up more waits behind it
  if (*reinterpret_cast<volatile int*>(&g_status_word) != 0) return;

  const uint32_t pad = (1024u - (smem_addr(smem_raw) & 1023u)) & 1023u;
  if (pad > (uint32_t)kPadAllowance) {                   // never seen; refuse rather than overrun
    if (tid == 0) atomicCAS(&g_status_word, 0, 90);
    return;
  }
  uint8_t* smem = smem_raw + pad;
  constexpr int kTiles = 1 + kNK + (HAS_V ? kNV : 0);
  PfShared& sh = *reinterpret_cast<PfShared*>(smem + kTiles * kStageBytes);
  uint64_t& bar_q = sh.bar_q;
  uint64_t* bar_kfull = sh.bar_kfull;
  uint64_t* bar_kempty = sh.bar_kempty;
  uint64_t* bar_vfull = sh.bar_vfull;
  uint64_t* bar_vempty = sh.bar_vempty;
  uint64_t* bar_sfull = sh.bar_sfull;
  uint64_t* bar_pready = sh.bar_pready;
  uint64_t* bar_odone = sh.bar_odone;
  uint64_t& bar_x = sh.bar_x;
  uint32_t& tmem_sh = sh.tmem;
  int& give_up = sh.give_up;
  float (&xchg)[2][2][128] = sh.xchg;
  float* lse_s = sh.xchg[0][1];                          // kPool only: that mode exchanges through xchg[.][0]
  const uint32_t q_s = smem_addr(smem);
  const uint32_t k_s = q_s + kStageBytes;
  const uint32_t v_s = k_s + kNK * kStageBytes;

  if (tid == 0) {
    mbar_init(&bar_q, 128);
    for (int i = 0; i < kNK; ++i) { mbar_init(&bar_kfull[i], 128); mbar_init(&bar_kempty[i], 1); }
    for (int i = 0; i < kNV; ++i) { mbar_init(&bar_vfull[i], 128); mbar_init(&bar_vempty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_sfull[i], 1);
      mbar_init(&bar_pready[i], 128);
      mbar_init(&bar_odone[i], 1);
    }
    mbar_init(&bar_x, kSoftmaxThreads);
    mbar_fence_init();
    give_up = 0;
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&tmem_sh, 512);
    tmem_relinquish();
  }
  if (POOL && tid < 128) {
    const int tok = tile_start + (tid >> 2);
    lse_s[tid] = tok < p.L ? p.lse2_in[((int64_t)b * p.L + tok) * p.H + g * kHg + (tid & 3)] : INFINITY;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_sh;
  const uint32_t t_s0 = tmem, t_o = tmem + 256;

  // Register budget per SM sub-partition (512 per thread slot, warps w, w+4, w+8, w+12 share one):
  // 2 x 200 (softmax) + 56 (producer) + 40 (MMA issuer / padding warp) = 496.
  if (warp >= kProducerWarp0 && warp < kMmaWarp) {
    // ================================ producers ================================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n");
    // Every thread copies with cp.async and lets the hardware arrive on the stage's "full" barrier when
    // its copies have landed (cp.async.mbarrier.arrive.noinc): the producers never wait for data, they
    // run ahead as far as the rings allow.  The MMA warp orders the landed bytes against the tensor
    // core's reads with a proxy fence after its barrier wait.
    const int pw = warp - kProducerWarp0, ptid = tid - kProducerWarp0 * 32;
    const __half* qb = p.q + (int64_t)b * p.q_sb;
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
      const int id = it * 128 + ptid, row = id >> 4, c = id & 15;
      const int tok = tile_start + (row >> 2), head = g * kHg + (row & 3);
      const bool in = tok < p.L;                         // rows past the prompt are zero-filled
      cp16_zfill(q_s + tile_off(row, c, 128),
                 qb + (int64_t)(in ? tok : 0) * p.q_st + (int64_t)head * p.q_sh + c * 8, in ? 16u : 0u);
    }
    cp_arrive_noinc(&bar_q);
    const __half* kb = p.k + (int64_t)b * p.k_sb + (int64_t)g * p.k_sh;
    const __half* vb = HAS_V ? p.v + (int64_t)b * p.v_sb + (int64_t)g * p.v_sh : nullptr;
    // key position of row (pw*32 + lane) of block j; index loads run two blocks ahead of their use
    auto load_key = [&](int j) -> int {
      const int s = j * 128 + pw * 32 + lane;
      if (j >= nb || s >= total) return 0;
      if (GATHER) return s < count ? __ldg(idx_row + s) : tile_start + (s - count);
      return s;
    };
    int key_a = load_key(0), key_b = load_key(1);
    for (int j = 0; j < nb; ++j) {
      int key = key_a;
      key_a = key_b;
      key_b = load_key(j + 2);
      key = max(0, min(key, p.L - 1));
      const int64_t offk = (int64_t)key * p.k_st;
      const int64_t offv = HAS_V ? (int64_t)key * p.v_st : 0;
      if (!mbar_wait(&bar_kempty[j % kNK], ((j / kNK) & 1) ^ 1, &give_up, 11)) break;
      {
        const uint32_t dst = k_s + (j % kNK) * kStageBytes;
        const int c = lane & 15;
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
          const int rw = it * 2 + (lane >> 4);
          const int64_t o = __shfl_sync(0xFFFFFFFFu, offk, rw);
          cp16(dst + tile_off(pw * 32 + rw, c, 128), kb + o + c * 8);
        }
        cp_arrive_noinc(&bar_kfull[j % kNK]);
      }
      if (HAS_V) {
        if (!mbar_wait(&bar_vempty[j % kNV], ((j / kNV) & 1) ^ 1, &give_up, 12)) break;
        const uint32_t dst = v_s + (j % kNV) * kStageBytes;
        const int c = lane & 15;
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
          const int rw = it * 2 + (lane >> 4);
          const int64_t o = __shfl_sync(0xFFFFFFFFu, offv, rw);
          cp16(dst + tile_off(pw * 32 + rw, c, 128), vb + o + c * 8);
        }
        cp_arrive_noinc(&bar_vfull[j % kNV]);
      }
    }
    cp_wait_all();                                       // nothing of this CTA is in flight at teardown
  } else if (warp >= kMmaWarp) {
    // ================================ MMA issuer (warp 12; warps 13-15 idle) ====================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;\n");
    if (warp == kMmaWarp && lane == 0) {
      constexpr uint32_t idesc_qk = idesc_f16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = idesc_f16(128, 128, 0, 1);
      bool ok = mbar_wait(&bar_q, 0, &give_up, 21);
      fence_proxy_async_smem();
      auto issue_qk = [&](int j) -> bool {
        if (!mbar_wait(&bar_kfull[j % kNK], (j / kNK) & 1, &give_up, 22)) return false;
        fence_proxy_async_smem();                        // cp.async bytes -> visible to the tensor core
        tc_fence_after();
        const uint32_t ks_addr = k_s + (j % kNK) * kStageBytes;
        const uint32_t d = t_s0 + (j & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * (kStageBytes / 2) + (ks & 3) * 32;
          const uint64_t dq = desc_kmajor(q_s + off), dk = desc_kmajor(ks_addr + off);
          if (POOL) mma_ss(d, dk, dq, idesc_qk, ks > 0);     // S^T: lanes = keys
          else mma_ss(d, dq, dk, idesc_qk, ks > 0);          // S: lanes = (query, head) rows
        }
        mma_commit(&bar_kempty[j % kNK]);
        mma_commit(&bar_sfull[j & 1]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) {
          if (!HAS_V && j >= 1) {
            ok = mbar_wait(&bar_pready[(j - 1) & 1], ((j - 1) >> 1) & 1, &give_up, 23);
            if (!ok) break;
          }
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        if (HAS_V) {
          ok = mbar_wait(&bar_pready[j & 1], (j >> 1) & 1, &give_up, 24);
          if (!ok) break;
          ok = mbar_wait(&bar_vfull[j % kNV], (j / kNV) & 1, &give_up, 25);
          if (!ok) break;
          fence_proxy_async_smem();
          tc_fence_after();
          const uint32_t vs_addr = v_s + (j % kNV) * kStageBytes;
          const uint32_t a = t_s0 + (j & 1) * 128;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            mma_ts(t_o + (j & 1) * 128, a + ks * 8, desc_mnmajor(vs_addr + ks * 2048, kStageBytes / 2), idesc_pv,
                   (j > 1 || ks > 0) ? 1u : 0u);
          }
          mma_commit(&bar_vempty[j % kNV]);
          mma_commit(&bar_odone[j & 1]);
        }
      }
    }
    __syncwarp();
  } else if (!POOL) {
    // ================================ softmax ==================================================
    // Two warpgroups, two independent streams: warpgroup w owns the key blocks j = w, w+2, ... with its
    // own S buffer, its own running (max, sum) per row and (with V) its own O accumulator, so the
    // tcgen05.ld / max / ex2 phases of one stream overlap those of the other and nothing is exchanged
    // per block.  The streams are merged like split-K partials in the epilogue.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;\n");
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane, q_local = row >> 2;
    const int tok = tile_start + q_local;
    const int off = GATHER ? count : tile_start;      // slot - off = key position inside the tile
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ts = t_s0 + wg * 128 + lane_sel;   // this stream's S / P buffer
    const uint32_t to = t_o + wg * 128 + lane_sel;    // this stream's O accumulator
    float m_run = -INFINITY, l_run = 0.f;             // m_run in the scaled (log2) domain
    bool ok = true;
    int it = 0;                                       // blocks this stream has processed
    for (int j = wg; j < nb; j += 2, ++it) {
      ok = mbar_wait(&bar_sfull[wg], it & 1, &give_up, 31);
      if (!ok) break;
      tc_fence_after();
      const int c0 = j * 128 - off;                     // key position (inside the tile) of column 0
      const bool need_mask = (c0 + 127) > 0;            // only the last block(s) of a tile
      // the whole S row (128 fp32) comes into registers with one round trip to tensor memory
      uint32_t sr[4][32];
#pragma unroll
      for (int part = 0; part < 4; ++part) tmem_ld32(ts + part * 32, sr[part]);
      tmem_wait_ld();
      if (!HAS_V) {                                      // S is in registers: the buffer may be refilled
        tc_fence_before();
        mbar_arrive(&bar_pready[wg]);
      }
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
      // than 2^kRescaleLog2: probabilities then stay below 2^kRescaleLog2 (exact in fp32, harmless in
      // fp16), and the O accumulator is rescaled only on those rare blocks.  lse2 = m + log2(l) holds
      // for any reference point m.
      const float m_new = (mx > m_run + kRescaleLog2) ? mx : m_run;
      const float alpha = ex2(m_run - m_new);
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      if (HAS_V) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t pr[32];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {              // P column i of this half = keys 2i, 2i+1
            const int c = half * 64 + i * 2;
            float a0 = ex2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), p.scale2, -m_new));
            float a1 = ex2(fmaf(__uint_as_float(sr[c >> 5][(c & 31) + 1]), p.scale2, -m_new));
            float a2 = ex2(fmaf(__uint_as_float(sr[c >> 5][(c & 31) + 2]), p.scale2, -m_new));
            float a3 = ex2(fmaf(__uint_as_float(sr[c >> 5][(c & 31) + 3]), p.scale2, -m_new));
            s0 += a0; s1 += a1; s2 += a2; s3 += a3;
            pr[i] = pack2(a0, a1);
            pr[i + 1] = pack2(a2, a3);
          }
          tmem_st32(ts + half * 32, pr);                 // P columns [half*32, +32) = keys [half*64, +64)
        }
      } else {
#pragma unroll
        for (int part = 0; part < 4; ++part)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            s0 += ex2(fmaf(__uint_as_float(sr[part][i]), p.scale2, -m_new));
            s1 += ex2(fmaf(__uint_as_float(sr[part][i + 1]), p.scale2, -m_new));
            s2 += ex2(fmaf(__uint_as_float(sr[part][i + 2]), p.scale2, -m_new));
            s3 += ex2(fmaf(__uint_as_float(sr[part][i + 3]), p.scale2, -m_new));
          }
      }
      l_run = l_run * alpha + ((s0 + s1) + (s2 + s3));
      m_run = m_new;
      if (HAS_V) {
        if (it > 0 && !__all_sync(0xFFFFFFFFu, alpha == 1.0f)) {
          // the previous P.V of this stream must have landed in O before O is rescaled
          ok = mbar_wait(&bar_odone[wg], (it - 1) & 1, &give_up, 32);
          if (!ok) break;
          tc_fence_after();
          {
#pragma unroll 1
            for (int part = 0; part < 4; ++part) {
              uint32_t orr[32];
              tmem_ld32(to + part * 32, orr);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
              tmem_st32(to + part * 32, orr);
            }
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bar_pready[wg]);
      }
    }
    // ---- epilogue: merge the two streams, normalise, store -------------------------------------
    // it = number of blocks of this stream; the other stream has nb - it
    float f_mine = 1.f, f_other = 0.f, l_tot = l_run, m_tot = m_run;
    if (ok) {
      xchg[0][wg][row] = m_run;
      xchg[1][wg][row] = l_run;
      mbar_arrive(&bar_x);
      ok = mbar_wait(&bar_x, 0, &give_up, 35);
      if (ok) {
        const float m_o = xchg[0][wg ^ 1][row], l_o = xchg[1][wg ^ 1][row];
        m_tot = fmaxf(m_run, m_o);
        f_mine = (m_run == -INFINITY) ? 0.f : ex2(m_run - m_tot);
        f_other = (m_o == -INFINITY) ? 0.f : ex2(m_o - m_tot);
        l_tot = l_run * f_mine + l_o * f_other;
      }
    }
    if (ok && HAS_V) {
      const int n_mine = it, n_other = nb - it;
      if (n_mine > 0) ok = mbar_wait(&bar_odone[wg], (n_mine - 1) & 1, &give_up, 33);
      if (ok && n_other > 0) ok = mbar_wait(&bar_odone[wg ^ 1], (n_other - 1) & 1, &give_up, 36);
      if (ok) {
        tc_fence_after();
        const float inv = 1.0f / l_tot;
        const float w_mine = f_mine * inv, w_other = f_other * inv;
        // this warpgroup stores output columns [wg*64, +64) of its rows, from both accumulators
        __half* orow = p.out + (((int64_t)b * p.L + tok) * p.H + g * kHg + (row & 3)) * kD + wg * 64;
        const uint32_t o_mine = t_o + wg * 128 + lane_sel + wg * 64;
        const uint32_t o_other = t_o + (wg ^ 1) * 128 + lane_sel + wg * 64;
#pragma unroll 1
        for (int part = 0; part < 2; ++part) {
          uint32_t oa[32], ob[32];
          if (n_mine > 0) tmem_ld32(o_mine + part * 32, oa);
          if (n_other > 0) tmem_ld32(o_other + part * 32, ob);
          tmem_wait_ld();
          if (tok < p.L) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float x = n_mine > 0 ? __uint_as_float(oa[i]) * w_mine : 0.f;
              if (n_other > 0) x = fmaf(__uint_as_float(ob[i]), w_other, x);
              v[i] = x;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = pack2(v[i * 8 + 0], v[i * 8 + 1]);
              w.y = pack2(v[i * 8 + 2], v[i * 8 + 3]);
              w.z = pack2(v[i * 8 + 4], v[i * 8 + 5]);
              w.w = pack2(v[i * 8 + 6], v[i * 8 + 7]);
              *reinterpret_cast<uint4*>(orow + part * 32 + i * 8) = w;
            }
          }
        }
      }
    }
    if (ok && wg == 0 && p.lse2 && tok < p.L)
      p.lse2[((int64_t)b * p.L + tok) * p.H + g * kHg + (row & 3)] = m_tot + log2f(l_tot);
  } else {
    // ================================ pooled-score reducer =====================================
    // warpgroup w owns the key blocks j = w, w+2, ...; thread = key lane, sums over the tile's 128
    // (query, head) rows, i.e. over the 128 columns of S^T
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;\n");
    const int wg = warp >> 2;
    const int key_lane = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ts = t_s0 + wg * 128 + lane_sel;
    float* prow = p.pooled + (((int64_t)b * p.G + g) * p.T + t) * p.pooled_stride;
    int it = 0;
    for (int j = wg; j < nb; j += 2, ++it) {
      if (!mbar_wait(&bar_sfull[wg], it & 1, &give_up, 41)) break;
      tc_fence_after();
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
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
          a0 += ex2(fmaf(__uint_as_float(sr[part][i]), p.scale2, -lse_s[part * 32 + i]));
          a1 += ex2(fmaf(__uint_as_float(sr[part][i + 1]), p.scale2, -lse_s[part * 32 + i + 1]));
          a2 += ex2(fmaf(__uint_as_float(sr[part][i + 2]), p.scale2, -lse_s[part * 32 + i + 2]));
          a3 += ex2(fmaf(__uint_as_float(sr[part][i + 3]), p.scale2, -lse_s[part * 32 + i + 3]));
        }
      const int key = j * 128 + key_lane;
      if (key < tile_start) prow[key] = (a0 + a1) + (a2 + a3);
    }
  }

  // ---- teardown: every role ends up here, also after a wait that gave up ----------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
  if (tid == 0 && give_up != 0) atomicCAS(&g_status_word, 0, give_up);
}

static_assert(sizeof(PfShared) <= 2304, "PfShared grew");
constexpr int kSmemAttn = kStageBytes * (1 + 3 + kNV) + kPadAllowance + 2304;   // = 232448, the sm_100 limit
constexpr int kSmemNoV = kStageBytes * (1 + kNKMax) + kPadAllowance + 2304;

int init_prefill() {
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kDenseAttn>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kSparse>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAttn));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kDenseLse>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemNoV));
  KB_CUDA(cudaFuncSetAttribute(tile_prefill_kernel<kPool>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemNoV));
  return 0;
}

static int fill_act(const kb200_act_layout* a, const __half** ptr, int64_t* sb, int64_t* st, int64_t* sh,
                    const char* what) {
  KB_REQUIRE(a && a->ptr, "prefill: %s is null", what);
  KB_REQUIRE((reinterpret_cast<uintptr_t>(a->ptr) & 15) == 0 && a->stride_b % 8 == 0 && a->stride_t % 8 == 0 &&
                 a->stride_h % 8 == 0,
             "prefill: %s must be 16-byte aligned with strides that are multiples of 8 elements", what);
  *ptr = static_cast<const __half*>(a->ptr);
  *sb = a->stride_b;
  *st = a->stride_t;
  *sh = a->stride_h;
  return 0;
}

static int check_shape(int batch, int seq_len, int H, int G) {
  KB_REQUIRE(initialised(nullptr), "kb200_init has not been called");
  KB_REQUIRE(batch >= 0 && seq_len >= 0, "prefill: negative size");
  KB_REQUIRE(G > 0 && H == G * kHg,
             "prefill: %d query heads / %d KV heads; exactly %d query heads per KV head are supported", H, G, kHg);
  KB_REQUIRE(batch <= 65535 && G <= 65535, "prefill: batch and KV heads must fit a grid dimension");
  return 0;
}

}  // namespace kb200

extern "C" int kb200_read_status(int* host_out) {
  using namespace kb200;
  KB_REQUIRE(host_out, "read_status: null pointer");
  int zero = 0;
  KB_CUDA(cudaMemcpyFromSymbol(host_out, g_status_word, sizeof(int)));
  KB_CUDA(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
  return 0;
}

extern "C" int kb200_prefill_dense(const kb200_act_layout* q, const kb200_act_layout* k,
                                   const kb200_act_layout* v, float softmax_scale, void* out, float* lse2,
                                   int batch, int seq_len, int num_q_heads, int num_kv_heads, void* stream) {
  using namespace kb200;
  if (check_shape(batch, seq_len, num_q_heads, num_kv_heads) != 0) return -1;
  KB_REQUIRE(out || lse2, "prefill_dense: nothing to compute (out and lse2 are both null)");
  if (batch == 0 || seq_len == 0) return 0;
  PrefillParams p{};
  if (fill_act(q, &p.q, &p.q_sb, &p.q_st, &p.q_sh, "q") != 0) return -1;
  if (fill_act(k, &p.k, &p.k_sb, &p.k_st, &p.k_sh, "k") != 0) return -1;
  if (out && fill_act(v, &p.v, &p.v_sb, &p.v_st, &p.v_sh, "v") != 0) return -1;
  KB_REQUIRE(!out || (reinterpret_cast<uintptr_t>(out) & 15) == 0, "prefill_dense: out must be 16-byte aligned");
  p.scale2 = softmax_scale * kLog2e;
  p.out = static_cast<__half*>(out);
  p.lse2 = lse2;
  p.B = batch; p.L = seq_len; p.H = num_q_heads; p.G = num_kv_heads; p.T = ceil_div(seq_len, kTile);
  dim3 grid(p.T, num_kv_heads, batch);
  if (out) tile_prefill_kernel<kDenseAttn><<<grid, kPfThreads, kSmemAttn, (cudaStream_t)stream>>>(p);
  else tile_prefill_kernel<kDenseLse><<<grid, kPfThreads, kSmemNoV, (cudaStream_t)stream>>>(p);
  KB_CHECK_LAUNCH("tile_prefill_kernel<dense>");
  return 0;
}

extern "C" int kb200_prefill_pool_scores(const kb200_act_layout* q, const kb200_act_layout* k,
                                         const float* lse2, float softmax_scale, float* pooled,
                                         int64_t row_stride, int batch, int seq_len, int num_q_heads,
                                         int num_kv_heads, void* stream) {
  using namespace kb200;
  if (check_shape(batch, seq_len, num_q_heads, num_kv_heads) != 0) return -1;
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
  dim3 grid(p.T, num_kv_heads, batch);
  tile_prefill_kernel<kPool><<<grid, kPfThreads, kSmemNoV, (cudaStream_t)stream>>>(p);
  KB_CHECK_LAUNCH("tile_prefill_kernel<pool>");
  return 0;
}

extern "C" int kb200_prefill_sparse(const kb200_act_layout* q, const kb200_act_layout* k,
                                    const kb200_act_layout* v, const int32_t* tile_idx, int64_t idx_stride,
                                    const int32_t* tile_count, const int32_t* head_map, float softmax_scale,
                                    void* out, float* lse2, int batch, int seq_len, int num_q_heads,
                                    int num_kv_heads, int idx_kv_heads, void* stream) {
  using namespace kb200;
  if (check_shape(batch, seq_len, num_q_heads, num_kv_heads) != 0) return -1;
  KB_REQUIRE(tile_idx && tile_count && out, "prefill_sparse: null pointer");
  KB_REQUIRE(idx_stride >= 0, "prefill_sparse: negative idx_stride");
  KB_REQUIRE(idx_kv_heads == 0 || head_map || idx_kv_heads == num_kv_heads,
             "prefill_sparse: idx_kv_heads differs from num_kv_heads, so a head_map is required");
  KB_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0, "prefill_sparse: out must be 16-byte aligned");
  if (batch == 0 || seq_len == 0) return 0;
  PrefillParams p{};
  if (fill_act(q, &p.q, &p.q_sb, &p.q_st, &p.q_sh, "q") != 0) return -1;
  if (fill_act(k, &p.k, &p.k_sb, &p.k_st, &p.k_sh, "k") != 0) return -1;
  if (fill_act(v, &p.v, &p.v_sb, &p.v_st, &p.v_sh, "v") != 0) return -1;
  p.tile_idx = tile_idx;
  p.G_idx = idx_kv_heads > 0 ? idx_kv_heads : num_kv_heads;
  p.idx_stride = idx_stride;
  p.tile_count = tile_count;
  p.head_map = head_map;
  p.scale2 = softmax_scale * kLog2e;
  p.out = static_cast<__half*>(out);
  p.lse2 = lse2;
  p.B = batch; p.L = seq_len; p.H = num_q_heads; p.G = num_kv_heads; p.T = ceil_div(seq_len, kTile);
  dim3 grid(p.T, num_kv_heads, batch);
  tile_prefill_kernel<kSparse><<<grid, kPfThreads, kSmemAttn, (cudaStream_t)stream>>>(p);
  KB_CHECK_LAUNCH("tile_prefill_kernel<sparse>");
  return 0;
}
