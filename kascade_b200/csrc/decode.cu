// Paged decode attention for Kascade: sparse (reuse layers) and dense (anchor layers).
//
// One query token per sequence, 4 query heads per KV head.  The work is HBM-bound: every selected
// (or, for anchors, every cached) key costs one 256-byte K row and one 256-byte V row.  A CTA owns
// one (sequence, KV head, split); each of its warps streams 16-key sub-tiles through a private
// cp.async ring (16-byte chunks, 16 lanes per row so a row is one contiguous 256-byte request) and
// feeds them to mma.sync m16n8k16 with the 4 query heads in rows 0..3 of the A operand.  Logical
// token positions are translated through the block table two sub-tiles ahead of the copy.
// Partials (m, l, O) of the warps are merged in shared memory, partials of the splits by a second
// small kernel.
//
// Replaces kernels/flash_decoding/reuse_kascade_gqa_decode.py:50-200 (gathered split-K decode and
// its combine) and recompute_kascade_gqa_decode.py:49-315 (dense split-K pass with raw-score dump,
// combine, per-KV-head pooled score).
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"

namespace kb200 {

constexpr int kDecWarps = 8;                                // warps of a full-size CTA (one per SM); half-size CTAs run two per SM
constexpr int kDecWarpsFp8 = 16;                           // FP8 rows are half as long: twice the warps in the same shared memory
constexpr int kDecStages = 3;
constexpr int kSub = 16;                                  // keys per sub-tile
constexpr int kDecStageBytes = kSub * kD * 2 * 2;         // K + V rows of one sub-tile
constexpr int kDecSmem = kDecWarps * kDecStages * kDecStageBytes;

struct DecodeParams {
  const __half* q;
  int64_t q_stride_b, q_stride_h;
  const __half* k;
  const __half* v;
  int64_t kv_stride_batch, kv_stride_page, kv_stride_token, kv_stride_head;
  const int32_t* block_table;
  int32_t block_table_stride;
  int32_t page_shift, page_mask;
  const int32_t* idx;            // sparse: index rows
  int64_t idx_stride_b, idx_stride_g;
  const int32_t* count;          // sparse: [B,G] valid entries (or NULL)
  int32_t k_max;
  const int32_t* head_map;       // sparse: [G] or NULL
  const int32_t* seq_lens;       // dense: [B]
  float scale2;                  // softmax_scale * log2(e)
  float* logits;                 // dense: [B,H,logit_stride]
  int64_t logit_stride;
  __half* out;                   // [B,H,D] (written here only when num_splits == 1)
  float* lse2;                   // [B,H]
  float* ws_m;                   // [B,H,S]
  float* ws_l;                   // [B,H,S]
  float* ws_o;                   // [B,H,S,D]
  int32_t H, G, num_splits;
  int32_t bf16;                  // host side: cache, q and the output are bf16, not fp16
  // FP8 (e4m3) cache: one fp32 scale per (page, KV head) for K and for V; q and the output are fp16
  int32_t fp8;
  const float* k_scale;
  const float* v_scale;
  int64_t sc_stride_batch, sc_stride_page, sc_stride_head;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void lds128(uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d, uint32_t addr) {
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// one output element in the storage type
template <bool BF16>
__device__ __forceinline__ void store_half(__half* dst, float x) {
  if (BF16) *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(x);
  else *dst = __float2half_rn(x);
}

// byte offset of 16-byte chunk `c` of row `r` inside a [16 rows x 256 B] sub-tile buffer
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4)); }

// two e4m3 values (16 bits) -> two fp16 values, exactly
__device__ __forceinline__ uint32_t fp8x2_to_half2(uint32_t two_bytes) {
  uint32_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}\n" : "=r"(r) : "r"(two_bytes));
  return r;
}

// byte offset of 16-byte chunk `c` of row `r` inside a [16 rows x 128 B] sub-tile buffer of FP8 rows
__device__ __forceinline__ uint32_t swz8(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// KV: storage of the cache.  0 fp16, 1 bf16 (q and the output have the same type), 2 FP8 e4m3 with one scale
// per (page, KV head).  FP8 rows of 128 bytes are copied as they are and the MMA operands are made from them in
// registers (cvt.rn.f16x2.e4m3x2, exact), without a second copy in shared memory:
//   * Q.K^T sums over d, so the order of d inside the MMAs is free: lane (key n, quad q) reads the 32 contiguous
//     bytes d = 32q .. 32q+31 of its key's row and uses 4 of them per k-step; the query fragments are loaded
//     with the same assignment.
//   * P.V needs pairs of keys per register: ldmatrix.trans over the bytes taken as 16-bit units gives
//     (V[2q][d], V[2q][d+1], V[2q+1][d], V[2q+1][d+1]); a byte permute splits that into the operand of the
//     even and of the odd columns, so a lane ends up with 4 contiguous d per 16-byte chunk.
// The scales are applied in fp32 where a row's contribution appears: on the logit of its key and on its
// probability before P.V.  q and the output are fp16 then.
constexpr int kRawStage = kSub * kD * 2;                  // FP8: K + V rows of a sub-tile as stored (4 KB)

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(x));
  return r;
}
// the two 16-bit halves of a word of e4m3 bytes -> two fp16 pairs
__device__ __forceinline__ void fp8x4_to_half2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}

__host__ __device__ constexpr int dec_warps(int kv) { return kv == 2 ? kDecWarpsFp8 : kDecWarps; }

// The MMAs run "transposed": the 16 keys of a sub-tile are the M rows, the query heads the N columns (4 of 8
// used), so that one m16n8k16 covers 16 keys x 16 d of Q.K^T and 16 d x 16 keys of P.V:
//   S^T[key][head] = K[key][d] . Q^T[d][head]        A = K rows (ldmatrix), B = the query fragments
//   O^T[d][head]   = V^T[d][key] . P^T[key][head]    A = V rows (ldmatrix.trans), B = P^T
// The C fragment of S^T holds (key g | g+8, heads 2q, 2q+1) per lane (g = lane / 4, q = lane % 4); packed to
// 16 bits and transposed with movmatrix it is the B fragment of P^T.  Lanes with q >= 2 carry the four unused
// columns (zero queries).  Running max and sum are per lane for its two heads; the sum stays a per-lane
// partial until the end.
template <bool DENSE, bool HAS_V, bool WRITE_LOGITS, int KV>
__global__ void __launch_bounds__(dec_warps(KV) * 32, 1) decode_attn_kernel(const DecodeParams p) {
  constexpr bool BF16 = KV == 1, FP8 = KV == 2;
  const int WARPS = blockDim.x >> 5;       // dec_warps(KV) or half of it, chosen at launch
  constexpr uint32_t FULL = 0xFFFFFFFFu;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 2;               // C fragment row: key grp (and grp + 8); B fragment column: head grp
  const int quad = lane & 3;               // C fragment columns: heads 2*quad, 2*quad + 1 (valid when quad < 2)

  // ---- this CTA's slice of the key list -----------------------------------------------------
  int n;
  const int32_t* idx_row = nullptr;
  if (DENSE) {
    n = p.seq_lens[b];
  } else {
    int src_g = p.head_map ? p.head_map[g] : g;
    n = p.count ? p.count[b * p.G + src_g] : p.k_max;
    n = min(n, p.k_max);
    idx_row = p.idx + b * p.idx_stride_b + src_g * p.idx_stride_g;
  }
  n = max(n, 0);
  const int nst = (n + kSub - 1) / kSub;
  const int per = (nst + p.num_splits - 1) / p.num_splits;
  const int st_begin = min(split * per, nst);
  const int st_end = min(st_begin + per, nst);
  // sub-tiles of this warp: st_begin + warp, + WARPS, ...
  const int my_count = (st_end - st_begin - warp + WARPS - 1) / WARPS;  // may be <= 0

  // ---- query fragments: B operand Q^T[d][head], column = head grp (zero for grp >= 4) ---------------
  uint32_t qb0[8], qb1[8];
  {
    const __half* qp = p.q + b * p.q_stride_b + (int64_t)(g * kHg + (grp & 3)) * p.q_stride_h;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      // FP8: k-step ks of quad q covers d = 32q + 4ks .. + 3 (the order of d inside the sum is free)
      uint32_t x0 = *reinterpret_cast<const uint32_t*>(qp + (FP8 ? quad * 32 + ks * 4 : ks * 16 + quad * 2));
      uint32_t x1 = *reinterpret_cast<const uint32_t*>(qp + (FP8 ? quad * 32 + ks * 4 + 2 : ks * 16 + 8 + quad * 2));
      qb0[ks] = grp < kHg ? x0 : 0u;
      qb1[ks] = grp < kHg ? x1 : 0u;
    }
  }

  const int64_t kv_base = (int64_t)b * p.kv_stride_batch + (int64_t)g * p.kv_stride_head;
  const int32_t* table = p.block_table ? p.block_table + (int64_t)b * p.block_table_stride : nullptr;
  constexpr int kStage = FP8 ? kRawStage : kDecStageBytes;
  uint8_t* my_smem = smem + warp * (kDecStages * kStage);
  const uint32_t my_smem_u32 = smem_u32(my_smem);

  // position of key `lane` (lanes 0..15) of sub-tile j of this warp, clamped into the list
  auto load_pos = [&](int j) -> int {
    int s = (st_begin + warp + j * WARPS) * kSub + (lane & 15);
    if (j >= my_count) return 0;
    s = min(s, n - 1);
    return DENSE ? s : __ldg(idx_row + s);
  };
  auto load_page = [&](int pos) -> int {
    int lp = pos >> p.page_shift;
    return table ? __ldg(table + lp) : lp;
  };
  auto issue = [&](int j, int pos, int page) {
    if (j < my_count) {
      int64_t off = kv_base + (int64_t)page * p.kv_stride_page +
                    (int64_t)(pos & p.page_mask) * p.kv_stride_token;
      const uint32_t dst = my_smem_u32 + (j % kDecStages) * kStage;
      if (FP8) {
        // rows of 128 bytes: 8 lanes per row, 4 rows per instruction, stored as they are
        const uint8_t* k8 = reinterpret_cast<const uint8_t*>(p.k);
        const uint8_t* v8 = reinterpret_cast<const uint8_t*>(p.v);
        const int c = lane & 7;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          int r = i * 4 + (lane >> 3);
          int64_t roff = __shfl_sync(FULL, off, r);
          cp_async16(dst + swz8(r, c), k8 + roff + c * 16);
          if (HAS_V) cp_async16(dst + kSub * kD + swz8(r, c), v8 + roff + c * 16);
        }
      } else {
        const int c = lane & 15;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          int r = i * 2 + (lane >> 4);
          int64_t roff = __shfl_sync(FULL, off, r);
          cp_async16(dst + swz(r, c), p.k + roff + c * 8);
          if (HAS_V) cp_async16(dst + kSub * kD * 2 + swz(r, c), p.v + roff + c * 8);
        }
      }
    }
    cp_async_commit();
  };
  // FP8: scales of the row this lane (0..15) stands for, from the page it lives in
  const int64_t sc_base = FP8 ? (int64_t)b * p.sc_stride_batch + (int64_t)g * p.sc_stride_head : 0;
  auto load_scale = [&](int page, float& sk, float& sv) {
    if (FP8) {
      const int64_t at = sc_base + (int64_t)page * p.sc_stride_page;
      sk = __ldg(p.k_scale + at);
      sv = HAS_V ? __ldg(p.v_scale + at) : 1.f;
    }
  };

  // ---- software pipeline: positions 2 ahead, pages 1 ahead, copies kDecStages-1 ahead ----------
  int pos_a = 0, page_a = 0, pos_b = 0;
  float sk0 = 1.f, sv0 = 1.f, sk1 = 1.f, sv1 = 1.f, sk2 = 1.f, sv2 = 1.f;   // FP8: scales of sub-tiles j, j+1, j+2
  {
    static_assert(kDecStages == 3, "the scale registers below assume two sub-tiles in flight");
    // all index loads first, then all page look-ups: the three dependent chains overlap
    const int pz0 = load_pos(0), pz1 = load_pos(1), pz2 = load_pos(2);
    const int pg0 = load_page(pz0), pg1 = load_page(pz1), pg2 = load_page(pz2);
    issue(0, pz0, pg0);
    load_scale(pg0, sk0, sv0);
    issue(1, pz1, pg1);
    load_scale(pg1, sk1, sv1);
    pos_a = pz2;
    page_a = pg2;
    pos_b = load_pos(kDecStages);
  }

  // O^T accumulators: o_acc[t][0|1] = (d_lo(t), heads 2q | 2q+1), o_acc[t][2|3] = (d_hi(t), ...) with
  // d_lo = 16t + grp, d_hi = d_lo + 8 (fp16 / bf16) or d_lo = 16t + 2 grp, d_hi = d_lo + 1 (FP8)
  float o_acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};

  for (int j = 0; j < my_count; ++j) {
    __syncwarp();                      // every lane is done with the buffer about to be refilled
    issue(j + kDecStages - 1, pos_a, page_a);
    load_scale(page_a, sk2, sv2);
    pos_a = pos_b;
    page_a = load_page(pos_a);
    pos_b = load_pos(j + kDecStages + 1);
    cp_async_wait<kDecStages - 1>();
    __syncwarp();

    const uint32_t kbuf = my_smem_u32 + (j % kDecStages) * kStage;
    const uint32_t vbuf = kbuf + kSub * kD * (FP8 ? 1 : 2);
    // ---- S^T = K Q^T : 8 k-steps, two accumulators to shorten the dependency chain ---------------
    float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
    if (FP8) {
      uint32_t wa[8], wb[8];                     // bytes d = 32q .. 32q+31 of key grp and of key grp + 8
      lds128(wa[0], wa[1], wa[2], wa[3], kbuf + swz8(grp, quad * 2));
      lds128(wa[4], wa[5], wa[6], wa[7], kbuf + swz8(grp, quad * 2 + 1));
      lds128(wb[0], wb[1], wb[2], wb[3], kbuf + swz8(grp + 8, quad * 2));
      lds128(wb[4], wb[5], wb[6], wb[7], kbuf + swz8(grp + 8, quad * 2 + 1));
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a0, a1, a2, a3;
        fp8x4_to_half2x2(wa[ks], a0, a2);
        fp8x4_to_half2x2(wb[ks], a1, a3);
        mma16816<false>((ks & 1) ? s2 : s, a0, a1, a2, a3, qb0[ks], qb1[ks]);
      }
    } else {
      // matrices of one ldmatrix.x4: (keys 0-7, chunk 2ks) (keys 8-15, 2ks) (keys 0-7, 2ks+1) (keys 8-15, 2ks+1)
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, kbuf + swz(r, ks * 2 + (lane >> 4)));
        mma16816<BF16>((ks & 1) ? s2 : s, a[0], a[1], a[2], a[3], qb0[ks], qb1[ks]);
      }
    }
    // ---- scale, mask the tail, dump logits ----------------------------------------------------
    const int key0 = (st_begin + warp + j * WARPS) * kSub;
    float x[4];                                  // (key grp, head 2q) (grp, 2q+1) (grp+8, 2q) (grp+8, 2q+1)
    {
      float fa = p.scale2, fb = p.scale2;
      if (FP8) {                                 // the key's own scale
        fa *= __shfl_sync(FULL, sk0, grp);
        fb *= __shfl_sync(FULL, sk0, grp + 8);
      }
      const bool va = key0 + grp < n, vb = key0 + grp + 8 < n;
      x[0] = va ? (s[0] + s2[0]) * fa : -INFINITY;
      x[1] = va ? (s[1] + s2[1]) * fa : -INFINITY;
      x[2] = vb ? (s[2] + s2[2]) * fb : -INFINITY;
      x[3] = vb ? (s[3] + s2[3]) * fb : -INFINITY;
      if (WRITE_LOGITS && quad < 2) {
        float* lp = p.logits + ((int64_t)b * p.H + g * kHg + quad * 2) * p.logit_stride + key0 + grp;
        if (va) { lp[0] = x[0]; lp[p.logit_stride] = x[1]; }
        if (vb) { lp[8] = x[2]; lp[p.logit_stride + 8] = x[3]; }
      }
    }
    float t0 = fmaxf(x[0], x[2]), t1 = fmaxf(x[1], x[3]);
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
      t0 = fmaxf(t0, __shfl_xor_sync(FULL, t0, sh));
      t1 = fmaxf(t1, __shfl_xor_sync(FULL, t1, sh));
    }
    const float m0 = fmaxf(m_run[0], t0), m1 = fmaxf(m_run[1], t1);   // finite: every sub-tile has >= 1 valid key
    const float alpha0 = exp2f(m_run[0] - m0), alpha1 = exp2f(m_run[1] - m1);
    m_run[0] = m0; m_run[1] = m1;
    float p0 = exp2f(x[0] - m0), p1 = exp2f(x[1] - m1), p2 = exp2f(x[2] - m0), p3 = exp2f(x[3] - m1);
    l_part[0] = l_part[0] * alpha0 + (p0 + p2);
    l_part[1] = l_part[1] * alpha1 + (p1 + p3);
    if (HAS_V) {
      if (FP8) {                                 // P.V sees the stored values: the rows' scales go on the probabilities
        const float va = __shfl_sync(FULL, sv0, grp), vb = __shfl_sync(FULL, sv0, grp + 8);
        p0 *= va; p1 *= va; p2 *= vb; p3 *= vb;
      }
      // B operand P^T[key][head]: column = head grp, rows = keys 2q, 2q+1 (b0) and 2q+8, 2q+9 (b1)
      const uint32_t pb0 = movmatrix_trans(pack_half2<BF16>(p0, p1));
      const uint32_t pb1 = movmatrix_trans(pack_half2<BF16>(p2, p3));
      // ---- O^T = O^T * alpha + V^T P^T : 8 d-tiles of 16 -----------------------------------------
      if (!__all_sync(FULL, alpha0 == 1.f && alpha1 == 1.f)) {         // a factor of exactly 1 changes nothing
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          o_acc[t][0] *= alpha0; o_acc[t][1] *= alpha1; o_acc[t][2] *= alpha0; o_acc[t][3] *= alpha1;
        }
      }
      if (FP8) {
        // ldmatrix.trans over the bytes as 16-bit units: lane gets (V[2q][d], V[2q][d+1], V[2q+1][d], V[2q+1][d+1]),
        // d = 16c + 2 grp; matrices of one x4: (keys 0-7, chunk 2t) (keys 8-15, 2t) (keys 0-7, 2t+1) (keys 8-15, 2t+1)
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int t2 = 0; t2 < 4; ++t2) {
          uint32_t rr[4];
          ldmatrix_x4_trans(rr, vbuf + swz8(r, t2 * 2 + (lane >> 4)));
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            // A rows 0-7: d = 16c + 2 grp (even bytes), rows 8-15: d + 1 (odd bytes); k = keys 2q.. (a0, a1), 2q+8.. (a2, a3)
            mma16816<false>(o_acc[t2 * 2 + h], fp8x2_to_half2(__byte_perm(rr[2 * h], 0u, 0x4420)),
                            fp8x2_to_half2(__byte_perm(rr[2 * h], 0u, 0x4431)),
                            fp8x2_to_half2(__byte_perm(rr[2 * h + 1], 0u, 0x4420)),
                            fp8x2_to_half2(__byte_perm(rr[2 * h + 1], 0u, 0x4431)), pb0, pb1);
          }
        }
      } else {
        // matrices of one ldmatrix.x4.trans: (keys 0-7, chunk 2t) (keys 0-7, 2t+1) (keys 8-15, 2t) (keys 8-15, 2t+1)
        const int r = (lane & 7) + (lane >> 4) * 8;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, vbuf + swz(r, t * 2 + ((lane >> 3) & 1)));
          mma16816<BF16>(o_acc[t], a[0], a[1], a[2], a[3], pb0, pb1);
        }
      }
    }
    if (FP8) { sk0 = sk1; sv0 = sv1; sk1 = sk2; sv1 = sv2; }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the warps of this CTA through shared memory ------------------------------------------
#pragma unroll
  for (int sh = 4; sh <= 16; sh <<= 1) {
    l_part[0] += __shfl_xor_sync(FULL, l_part[0], sh);
    l_part[1] += __shfl_xor_sync(FULL, l_part[1], sh);
  }
  float* sm_m = reinterpret_cast<float*>(smem);                  // [warps][4]
  float* sm_l = sm_m + WARPS * kHg;                              // [warps][4]
  float* sm_o = sm_l + WARPS * kHg;                              // [warps][4][128]
  if (quad < 2) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int h = quad * 2 + e;
      if (grp == 0) { sm_m[warp * kHg + h] = m_run[e]; sm_l[warp * kHg + h] = l_part[e]; }
      if (HAS_V) {
        float* dst = sm_o + (warp * kHg + h) * kD;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int d_lo = FP8 ? t * 16 + grp * 2 : t * 16 + grp;
          dst[d_lo] = o_acc[t][e];
          dst[d_lo + (FP8 ? 1 : 8)] = o_acc[t][2 + e];
        }
      }
    }
  }
  __syncthreads();
  for (int t = threadIdx.x; t < kHg * kD; t += WARPS * 32) {
    const int h = t / kD, d = t % kD;
    float M = -INFINITY;
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w * kHg + h]);
    float L = 0.f, O = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      float mw = sm_m[w * kHg + h];
      float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += sm_l[w * kHg + h] * f;
      if (HAS_V) O += sm_o[(w * kHg + h) * kD + d] * f;
    }
    const int64_t bh = (int64_t)b * p.H + g * kHg + h;
    if (p.num_splits == 1) {
      if (HAS_V) store_half<BF16>(p.out + bh * kD + d, L > 0.f ? O / L : 0.f);
      if (d == 0 && p.lse2) p.lse2[bh] = L > 0.f ? M + log2f(L) : -INFINITY;
    } else {
      const int64_t slot = bh * p.num_splits + split;
      if (HAS_V) p.ws_o[slot * kD + d] = O;
      if (d == 0) { p.ws_m[slot] = M; p.ws_l[slot] = L; }
    }
  }
}

// merge the split partials: grid (H, B), 128 threads (one per output element)
template <bool HAS_V, bool BF16>
__global__ void __launch_bounds__(kD) decode_combine_kernel(const float* __restrict__ ws_m,
                                                            const float* __restrict__ ws_l,
                                                            const float* __restrict__ ws_o,
                                                            __half* __restrict__ out,
                                                            float* __restrict__ lse2, int H,
                                                            int num_splits) {
  const int64_t bh = (int64_t)blockIdx.y * H + blockIdx.x;
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, ws_m[bh * num_splits + s]);
  float L = 0.f, O = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    float ms = ws_m[bh * num_splits + s];
    float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += ws_l[bh * num_splits + s] * f;
    if (HAS_V) O += ws_o[(bh * num_splits + s) * kD + d] * f;
  }
  if (HAS_V) store_half<BF16>(out + bh * kD + d, L > 0.f ? O / L : 0.f);
  if (d == 0 && lse2) lse2[bh] = L > 0.f ? M + log2f(L) : -INFINITY;
}

// pooled[b,g,j] = sum_h exp2(logit[b,4g+h,j] - lse2[b,4g+h]); grid (ceil(maxlen/1024), G, B)
__global__ void __launch_bounds__(256) decode_pool_kernel(const float* __restrict__ logits,
                                                          const float* __restrict__ lse2,
                                                          const int32_t* __restrict__ seq_lens,
                                                          float* __restrict__ pooled,
                                                          int64_t stride, int H, int G) {
  const int b = blockIdx.z, g = blockIdx.y;
  const int n = seq_lens[b];
  const int j = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (j >= n) return;
  float l[kHg];
#pragma unroll
  for (int h = 0; h < kHg; ++h) l[h] = lse2[(int64_t)b * H + g * kHg + h];
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int h = 0; h < kHg; ++h) {
    const float* src = logits + ((int64_t)b * H + g * kHg + h) * stride + j;
    float4 x = *reinterpret_cast<const float4*>(src);   // padding beyond n is readable scratch
    acc.x += exp2f(x.x - l[h]);
    acc.y += exp2f(x.y - l[h]);
    acc.z += exp2f(x.z - l[h]);
    acc.w += exp2f(x.w - l[h]);
  }
  float* dst = pooled + ((int64_t)b * G + g) * stride + j;
  if (j + 3 < n) {
    *reinterpret_cast<float4*>(dst) = acc;
  } else {
    float a[4] = {acc.x, acc.y, acc.z, acc.w};
    for (int e = 0; e < 4 && j + e < n; ++e) dst[e] = a[e];
  }
}

int init_decode() {
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<false, true, false, 0>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<true, true, true, 0>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<true, false, true, 0>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<false, true, false, 1>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<true, true, true, 1>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<true, false, true, 1>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<false, true, false, 2>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<true, true, true, 2>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  KB_CUDA(cudaFuncSetAttribute(decode_attn_kernel<true, false, true, 2>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem));
  return 0;
}

// Launch of the attention kernel.  Full-size CTAs (8 warps, 16 for an FP8 cache: 192 KB of copy rings, one CTA
// per SM) while the grid is small; half-size CTAs, two per SM, once the grid is at least 1.5 x the SMs: then one
// CTA's start (index -> block table -> row chain) and merge overlap the other's stream, which measured 3-9 %
// faster at batch 32-64 and 5-10 % slower at batch <= 16.
#ifndef KB200_DEC_HALF_FROM
#define KB200_DEC_HALF_FROM 3      // half-size CTAs from this many CTAs per two SMs on
#endif
template <bool DENSE, bool HAS_V, bool WRITE_LOGITS, int KV>
static void launch_attn(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  const long long total = (long long)grid.x * grid.y * grid.z;
  const int warps = total * 2 >= (long long)KB200_DEC_HALF_FROM * sm_count() ? dec_warps(KV) / 2 : dec_warps(KV);
  const size_t smem = (size_t)warps * kDecStages * (KV == 2 ? kRawStage : kDecStageBytes);
  decode_attn_kernel<DENSE, HAS_V, WRITE_LOGITS, KV><<<grid, warps * 32, smem, st>>>(p);
}

static int fill_kv(DecodeParams& p, const kb200_kv_layout* kv, bool need_v) {
  KB_REQUIRE(kv && kv->k, "decode: null KV layout");
  KB_REQUIRE(!need_v || kv->v, "decode: value cache required");
  KB_REQUIRE(kv->page_size >= 1 && (kv->page_size & (kv->page_size - 1)) == 0,
             "decode: page_size (%d) must be a power of two", kv->page_size);
  KB_REQUIRE((reinterpret_cast<uintptr_t>(kv->k) & 15) == 0 &&
                 (!kv->v || (reinterpret_cast<uintptr_t>(kv->v) & 15) == 0),
             "decode: KV cache must be 16-byte aligned");
  KB_REQUIRE(kv->stride_batch % 8 == 0 && kv->stride_page % 8 == 0 && kv->stride_token % 8 == 0 &&
                 kv->stride_head % 8 == 0,
             "decode: KV strides must be multiples of 8 elements (16 bytes)");
  KB_REQUIRE(kv->dtype == KB200_FP16 || kv->dtype == KB200_BF16 || kv->dtype == KB200_FP8_E4M3,
             "decode: unknown dtype code %d of the KV cache", kv->dtype);
  p.bf16 = kv->dtype == KB200_BF16;
  p.fp8 = kv->dtype == KB200_FP8_E4M3;
  if (p.fp8) {
    KB_REQUIRE(kv->k_scale && (!need_v || kv->v_scale), "decode: an FP8 cache needs k_scale / v_scale");
    KB_REQUIRE(kv->stride_batch % 16 == 0 && kv->stride_page % 16 == 0 && kv->stride_token % 16 == 0 &&
                   kv->stride_head % 16 == 0,
               "decode: strides of an FP8 cache must be multiples of 16 elements (16 bytes)");
    p.k_scale = kv->k_scale;
    p.v_scale = kv->v_scale;
    p.sc_stride_batch = kv->scale_stride_batch;
    p.sc_stride_page = kv->scale_stride_page;
    p.sc_stride_head = kv->scale_stride_head;
  }
  p.k = static_cast<const __half*>(kv->k);
  p.v = static_cast<const __half*>(kv->v);
  p.kv_stride_batch = kv->stride_batch;
  p.kv_stride_page = kv->stride_page;
  p.kv_stride_token = kv->stride_token;
  p.kv_stride_head = kv->stride_head;
  p.block_table = kv->block_table;
  p.block_table_stride = kv->block_table_stride;
  int shift = 0;
  while ((1 << shift) < kv->page_size) ++shift;
  p.page_shift = shift;
  p.page_mask = kv->page_size - 1;
  return 0;
}

// Splits per (sequence, KV head): as many as it takes to put about one CTA on every SM, and none beyond that -
// a CTA has a fixed cost (pipeline fill, merge of its warps, the partials and their combine pass) that measured
// larger than what a second wave of smaller CTAs gains.  At least 256 keys per split.
static int default_splits(int batch, int G, int max_keys) {
  int64_t ctas = (int64_t)batch * G;
  if (ctas <= 0) return 1;
  int want = (int)(sm_count() / ctas);
  int cap = max_keys / 256;
  if (cap < 1) cap = 1;
  int s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

static int set_workspace(DecodeParams& p, void* ws, size_t ws_bytes, int batch, int H, int splits) {
  size_t need = kb200_decode_workspace_bytes(batch, H, splits);
  KB_REQUIRE(splits == 1 || (ws && ws_bytes >= need),
             "decode: workspace of %zu bytes required, got %zu", need, ws_bytes);
  KB_REQUIRE(splits == 1 || (reinterpret_cast<uintptr_t>(ws) & 15) == 0,
             "decode: workspace must be 16-byte aligned");
  float* f = static_cast<float*>(ws);
  size_t bhs = (size_t)batch * H * splits;
  p.ws_m = f;
  p.ws_l = f + bhs;
  p.ws_o = f + 2 * bhs;
  return 0;
}

// ---- scratch that lives inside the library image (for kb200_decode_sparse_paged_noalloc) ------------
// Split partials of one call: KB200_NOALLOC_MAX_SLOTS slots of (m, l, O[128]) fp32.  Every GPU that
// loads the library carries this array until the process exits.
static __device__ __align__(256) float g_static_partials[KB200_NOALLOC_MAX_SLOTS * (2 + KB200_HEAD_DIM)];

constexpr int kMaxDevices = 64;
static float* g_static_ptr[kMaxDevices] = {};
static std::mutex g_static_mutex;

// Device address of g_static_partials on the CURRENT device.  In host code the array's name is only a
// handle for the runtime, not something a kernel may dereference, so the address is looked up once
// per device with cudaGetSymbolAddress and cached.
static int static_partials(float** out) {
  int dev = -1;
  KB_CUDA(cudaGetDevice(&dev));
  KB_REQUIRE(dev >= 0 && dev < kMaxDevices, "decode_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    float* ptr = nullptr;
    KB_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_partials));
    KB_REQUIRE(ptr != nullptr, "decode_noalloc: cudaGetSymbolAddress returned a null address");
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return 0;
}

// Splits the no-allocation entry point uses: an explicit request as given if it fits the built-in scratch
// (a single split always fits, it needs none), the library's own choice lowered until it fits; 0 = rejected.
static int noalloc_splits(int batch, int H, int G, int k_max, int num_splits) {
  int splits = num_splits > 0 ? num_splits : default_splits(batch, G, k_max);
  if (num_splits == 0)
    while (splits > 1 && (long long)batch * H * splits > KB200_NOALLOC_MAX_SLOTS) --splits;
  if (splits > 1 && (long long)batch * H * splits > KB200_NOALLOC_MAX_SLOTS) return 0;
  return splits;
}

}  // namespace kb200

extern "C" int kb200_decode_noalloc_splits(int batch, int num_q_heads, int num_kv_heads, int k_max, int num_splits) {
  if (batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_splits < 0) return 0;
  return kb200::noalloc_splits(batch, num_q_heads, num_kv_heads, k_max, num_splits);
}

extern "C" size_t kb200_decode_workspace_bytes(int batch, int num_q_heads, int num_splits) {
  if (batch <= 0 || num_q_heads <= 0 || num_splits <= 0) return 0;
  return (size_t)batch * num_q_heads * num_splits * (2 + KB200_HEAD_DIM) * sizeof(float);
}

extern "C" int kb200_decode_default_splits(int batch, int num_kv_heads, int max_keys) {
  return kb200::default_splits(batch, num_kv_heads, max_keys);
}

extern "C" int kb200_decode_sparse_paged(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                         const kb200_kv_layout* kv, const int32_t* topk_idx,
                                         int64_t idx_stride_b, int64_t idx_stride_g,
                                         const int32_t* topk_count, int k_max,
                                         const int32_t* head_map, float softmax_scale, void* out,
                                         float* lse2_out, void* workspace, size_t workspace_bytes,
                                         int batch, int num_q_heads, int num_kv_heads,
                                         int num_splits, void* stream) {
  using namespace kb200;
  KB_ENTRY(q, "decode_sparse: q");
  KB_REQUIRE(q && topk_idx && out, "decode_sparse: null pointer");
  KB_REQUIRE(batch >= 0 && k_max >= 0, "decode_sparse: negative size");
  KB_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * kHg,
             "decode_sparse: %d query heads / %d KV heads; exactly %d query heads per KV head are supported",
             num_q_heads, num_kv_heads, kHg);
  KB_REQUIRE(q_stride_h % 2 == 0 && q_stride_b % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0,
             "decode_sparse: q must be 4-byte aligned with even strides");
  KB_REQUIRE(num_splits >= 0 && num_splits <= 64, "decode_sparse: num_splits out of range");
  if (batch == 0) return 0;
  DecodeParams p{};
  if (fill_kv(p, kv, true) != 0) return -1;
  int splits = num_splits > 0 ? num_splits : default_splits(batch, num_kv_heads, k_max);
  if (set_workspace(p, workspace, workspace_bytes, batch, num_q_heads, splits) != 0) return -1;
  p.q = static_cast<const __half*>(q);
  p.q_stride_b = q_stride_b;
  p.q_stride_h = q_stride_h;
  p.idx = topk_idx;
  p.idx_stride_b = idx_stride_b;
  p.idx_stride_g = idx_stride_g;
  p.count = topk_count;
  p.k_max = k_max;
  p.head_map = head_map;
  p.scale2 = softmax_scale * kLog2e;
  p.out = static_cast<__half*>(out);
  p.lse2 = lse2_out;
  p.H = num_q_heads;
  p.G = num_kv_heads;
  p.num_splits = splits;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(splits, num_kv_heads, batch);
  if (p.fp8) launch_attn<false, true, false, 2>(p, grid, st);
  else if (p.bf16) launch_attn<false, true, false, 1>(p, grid, st);
  else launch_attn<false, true, false, 0>(p, grid, st);
  KB_CHECK_LAUNCH("decode_attn_kernel<sparse>");
  if (splits > 1) {
    if (p.bf16)
      decode_combine_kernel<true, true><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                 num_q_heads, splits);
    else
      decode_combine_kernel<true, false><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                  num_q_heads, splits);
    KB_CHECK_LAUNCH("decode_combine_kernel");
  }
  return 0;
}

extern "C" int kb200_decode_anchor_paged(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                         const kb200_kv_layout* kv, const int32_t* seq_lens,
                                         int max_seq_len, float softmax_scale, float* logits,
                                         float* pooled, int64_t logit_stride, void* out,
                                         float* lse2_out, void* workspace, size_t workspace_bytes,
                                         int batch, int num_q_heads, int num_kv_heads,
                                         int num_splits, void* stream) {
  using namespace kb200;
  KB_ENTRY(q, "decode_anchor: q");
  KB_REQUIRE(q && seq_lens && logits && pooled && lse2_out, "decode_anchor: null pointer");
  KB_REQUIRE(batch >= 0 && max_seq_len >= 0, "decode_anchor: negative size");
  KB_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * kHg,
             "decode_anchor: %d query heads / %d KV heads; exactly %d query heads per KV head are supported",
             num_q_heads, num_kv_heads, kHg);
  KB_REQUIRE(logit_stride % 4 == 0 && logit_stride >= ((max_seq_len + 3) & ~3),
             "decode_anchor: logit_stride (%lld) must be a multiple of 4 covering max_seq_len (%d)",
             (long long)logit_stride, max_seq_len);
  KB_REQUIRE((reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(pooled) & 15) == 0,
             "decode_anchor: logits / pooled must be 16-byte aligned");
  KB_REQUIRE(q_stride_h % 2 == 0 && q_stride_b % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0,
             "decode_anchor: q must be 4-byte aligned with even strides");
  KB_REQUIRE(num_splits >= 0 && num_splits <= 64, "decode_anchor: num_splits out of range");
  if (batch == 0) return 0;
  const bool has_v = out != nullptr;
  DecodeParams p{};
  if (fill_kv(p, kv, has_v) != 0) return -1;
  int splits = num_splits > 0 ? num_splits : default_splits(batch, num_kv_heads, max_seq_len);
  if (set_workspace(p, workspace, workspace_bytes, batch, num_q_heads, splits) != 0) return -1;
  p.q = static_cast<const __half*>(q);
  p.q_stride_b = q_stride_b;
  p.q_stride_h = q_stride_h;
  p.seq_lens = seq_lens;
  p.scale2 = softmax_scale * kLog2e;
  p.logits = logits;
  p.logit_stride = logit_stride;
  p.out = static_cast<__half*>(out);
  p.lse2 = lse2_out;
  p.H = num_q_heads;
  p.G = num_kv_heads;
  p.num_splits = splits;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(splits, num_kv_heads, batch);
  if (has_v && p.fp8) launch_attn<true, true, true, 2>(p, grid, st);
  else if (has_v && p.bf16) launch_attn<true, true, true, 1>(p, grid, st);
  else if (has_v) launch_attn<true, true, true, 0>(p, grid, st);
  else if (p.fp8) launch_attn<true, false, true, 2>(p, grid, st);
  else if (p.bf16) launch_attn<true, false, true, 1>(p, grid, st);
  else launch_attn<true, false, true, 0>(p, grid, st);
  KB_CHECK_LAUNCH("decode_attn_kernel<dense>");
  if (splits > 1) {
    if (has_v && p.bf16)
      decode_combine_kernel<true, true><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                 num_q_heads, splits);
    else if (has_v)
      decode_combine_kernel<true, false><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                  num_q_heads, splits);
    else
      decode_combine_kernel<false, false><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                   num_q_heads, splits);
    KB_CHECK_LAUNCH("decode_combine_kernel");
  }
  if (max_seq_len > 0) {
    dim3 pgrid(ceil_div(max_seq_len, 1024), num_kv_heads, batch);
    decode_pool_kernel<<<pgrid, 256, 0, st>>>(logits, lse2_out, seq_lens, pooled, logit_stride,
                                              num_q_heads, num_kv_heads);
    KB_CHECK_LAUNCH("decode_pool_kernel");
  }
  return 0;
}

// Same computation as kb200_decode_sparse_paged, for callers that must not allocate device memory and
// have no workspace to hand over: the split partials go to an array inside the library image.
extern "C" int kb200_decode_sparse_paged_noalloc(const void* q, int64_t q_stride_b, int64_t q_stride_h,
                                                 const kb200_kv_layout* kv, const int32_t* topk_idx,
                                                 int64_t idx_stride_b, int64_t idx_stride_g,
                                                 const int32_t* topk_count, int k_max,
                                                 const int32_t* head_map, float softmax_scale, void* out,
                                                 float* lse2_out, int batch, int num_q_heads,
                                                 int num_kv_heads, int num_splits, void* stream) {
  using namespace kb200;
  KB_ENTRY(q, "decode_noalloc: q");
  KB_REQUIRE(q && topk_idx && out, "decode_noalloc: null pointer");
  KB_REQUIRE(batch >= 0 && k_max >= 0, "decode_noalloc: negative size");
  KB_REQUIRE(num_kv_heads > 0 && num_q_heads == num_kv_heads * kHg,
             "decode_noalloc: %d query heads / %d KV heads; exactly %d query heads per KV head are supported",
             num_q_heads, num_kv_heads, kHg);
  KB_REQUIRE(q_stride_h % 2 == 0 && q_stride_b % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0,
             "decode_noalloc: q must be 4-byte aligned with even strides");
  KB_REQUIRE(num_splits >= 0 && num_splits <= 64, "decode_noalloc: num_splits out of range");
  if (batch == 0) return 0;
  DecodeParams p{};
  if (fill_kv(p, kv, true) != 0) return -1;
  const int splits = noalloc_splits(batch, num_q_heads, num_kv_heads, k_max, num_splits);
  const long long slots = (long long)batch * num_q_heads * (splits > 0 ? splits : num_splits);
  KB_REQUIRE(splits > 0,
             "decode_noalloc: batch %d x %d heads x %d splits = %lld partial slots exceed the built-in scratch of %d "
             "slots; use fewer splits or kb200_decode_sparse_paged with a caller-owned workspace",
             batch, num_q_heads, num_splits, slots, KB200_NOALLOC_MAX_SLOTS);
  if (splits > 1) {                            // a single split writes the output directly: no scratch, no look-up
    float* scratch = nullptr;
    if (static_partials(&scratch) != 0) return -1;
    const size_t bhs = (size_t)batch * num_q_heads * splits;
    p.ws_m = scratch;
    p.ws_l = scratch + bhs;
    p.ws_o = scratch + 2 * bhs;
  }
  p.q = static_cast<const __half*>(q);
  p.q_stride_b = q_stride_b;
  p.q_stride_h = q_stride_h;
  p.idx = topk_idx;
  p.idx_stride_b = idx_stride_b;
  p.idx_stride_g = idx_stride_g;
  p.count = topk_count;
  p.k_max = k_max;
  p.head_map = head_map;
  p.scale2 = softmax_scale * kLog2e;
  p.out = static_cast<__half*>(out);
  p.lse2 = lse2_out;
  p.H = num_q_heads;
  p.G = num_kv_heads;
  p.num_splits = splits;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(splits, num_kv_heads, batch);
  if (p.fp8) launch_attn<false, true, false, 2>(p, grid, st);
  else if (p.bf16) launch_attn<false, true, false, 1>(p, grid, st);
  else launch_attn<false, true, false, 0>(p, grid, st);
  KB_CHECK_LAUNCH("decode_attn_kernel<sparse, noalloc>");
  if (splits > 1) {
    if (p.bf16)
      decode_combine_kernel<true, true><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                 num_q_heads, splits);
    else
      decode_combine_kernel<true, false><<<dim3(num_q_heads, batch), kD, 0, st>>>(p.ws_m, p.ws_l, p.ws_o, p.out, p.lse2,
                                                                                  num_q_heads, splits);
    KB_CHECK_LAUNCH("decode_combine_kernel<noalloc>");
  }
  return 0;
}
