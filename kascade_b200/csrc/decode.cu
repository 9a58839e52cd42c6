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

constexpr int kDecWarps = 8;
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

// KV: storage of the cache.  0 fp16, 1 bf16 (q and the output have the same type), 2 FP8 e4m3 with one scale
// per (page, KV head): rows of 128 bytes are copied as they are, turned into fp16 in shared memory (exact), and
// the scales are applied in fp32 where a row's contribution appears: on the logit of its key and on its
// probability before P.V.  q and the output are fp16 then.
constexpr int kRawStage = kSub * kD * 2;                  // FP8: K + V rows of a sub-tile as stored (4 KB)
constexpr int kWarpSmemFp8 = kDecStages * kRawStage + kDecStageBytes;   // three raw stages + one fp16 working copy

template <bool DENSE, bool HAS_V, bool WRITE_LOGITS, int KV>
__global__ void __launch_bounds__(kDecWarps * 32, 1) decode_attn_kernel(const DecodeParams p) {
  constexpr bool BF16 = KV == 1, FP8 = KV == 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_head = lane >> 2;          // A/C fragment row = query head (valid when < 4)
  const int quad = lane & 3;

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
  // sub-tiles of this warp: st_begin + warp, + kDecWarps, ...
  const int my_count = (st_end - st_begin - warp + kDecWarps - 1) / kDecWarps;  // may be <= 0

  // ---- query fragments (rows 0..3 = heads, rows 4..15 zero) ----------------------------------
  uint32_t qa0[8], qa2[8];
  {
    const __half* qp = p.q + b * p.q_stride_b + (int64_t)(g * kHg + (row_head & 3)) * p.q_stride_h;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t x0 = *reinterpret_cast<const uint32_t*>(qp + ks * 16 + quad * 2);
      uint32_t x2 = *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + quad * 2);
      qa0[ks] = row_head < kHg ? x0 : 0u;
      qa2[ks] = row_head < kHg ? x2 : 0u;
    }
  }

  const int64_t kv_base = (int64_t)b * p.kv_stride_batch + (int64_t)g * p.kv_stride_head;
  const int32_t* table = p.block_table ? p.block_table + (int64_t)b * p.block_table_stride : nullptr;
  uint8_t* my_smem = smem + warp * (FP8 ? kWarpSmemFp8 : kDecStages * kDecStageBytes);
  const uint32_t my_smem_u32 = smem_u32(my_smem);
  const uint32_t work_u32 = my_smem_u32 + kDecStages * kRawStage;       // FP8: the fp16 copy the MMAs read

  // position of key `lane` (lanes 0..15) of sub-tile j of this warp, clamped into the list
  auto load_pos = [&](int j) -> int {
    int s = (st_begin + warp + j * kDecWarps) * kSub + (lane & 15);
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
      if (FP8) {
        // rows of 128 bytes: 8 lanes per row, 4 rows per instruction, stored as they are
        const uint32_t dst = my_smem_u32 + (j % kDecStages) * kRawStage;
        const uint8_t* k8 = reinterpret_cast<const uint8_t*>(p.k);
        const uint8_t* v8 = reinterpret_cast<const uint8_t*>(p.v);
        const int c = lane & 7;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          int r = i * 4 + (lane >> 3);
          int64_t roff = __shfl_sync(0xFFFFFFFFu, off, r);
          cp_async16(dst + r * 128 + c * 16, k8 + roff + c * 16);
          if (HAS_V) cp_async16(dst + kSub * kD + r * 128 + c * 16, v8 + roff + c * 16);
        }
      } else {
        uint32_t dst = my_smem_u32 + (j % kDecStages) * kDecStageBytes;
        const int c = lane & 15;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          int r = i * 2 + (lane >> 4);
          int64_t roff = __shfl_sync(0xFFFFFFFFu, off, r);
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
  // prologue
  {
    int pz = load_pos(0);
    int pgz = load_page(pz);
    pos_a = pz; page_a = pgz;
    static_assert(kDecStages == 3, "the scale registers below assume two sub-tiles in flight");
    issue(0, pos_a, page_a);
    load_scale(page_a, sk0, sv0);
    pos_a = load_pos(1);
    page_a = load_page(pos_a);
    issue(1, pos_a, page_a);
    load_scale(page_a, sk1, sv1);
    pos_a = load_pos(2);
    page_a = load_page(pos_a);
    pos_b = load_pos(kDecStages);
  }

  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run = -INFINITY, l_run = 0.f;   // per head (row_head), replicated over the quad

  for (int j = 0; j < my_count; ++j) {
    __syncwarp();                      // every lane is done with the buffer about to be refilled
    issue(j + kDecStages - 1, pos_a, page_a);
    load_scale(page_a, sk2, sv2);
    pos_a = pos_b;
    page_a = load_page(pos_a);
    pos_b = load_pos(j + kDecStages + 1);
    cp_async_wait<kDecStages - 1>();
    __syncwarp();

    if (FP8) {
      // the sub-tile as stored -> fp16 in the layout the fragment loads expect (16 bytes -> two 16-byte chunks)
      const uint8_t* raw = my_smem + (j % kDecStages) * kRawStage;
      const int c = lane & 7;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 4 + (lane >> 3);
#pragma unroll
        for (int kv = 0; kv < (HAS_V ? 2 : 1); ++kv) {
          const uint4 x = *reinterpret_cast<const uint4*>(raw + kv * kSub * kD + r * 128 + c * 16);
          uint4 lo, hi;
          lo.x = fp8x2_to_half2(x.x); lo.y = fp8x2_to_half2(x.x >> 16);
          lo.z = fp8x2_to_half2(x.y); lo.w = fp8x2_to_half2(x.y >> 16);
          hi.x = fp8x2_to_half2(x.z); hi.y = fp8x2_to_half2(x.z >> 16);
          hi.z = fp8x2_to_half2(x.w); hi.w = fp8x2_to_half2(x.w >> 16);
          uint8_t* dst = my_smem + kDecStages * kRawStage + kv * kSub * kD * 2;
          *reinterpret_cast<uint4*>(dst + swz(r, 2 * c)) = lo;
          *reinterpret_cast<uint4*>(dst + swz(r, 2 * c + 1)) = hi;
        }
      }
      __syncwarp();
    }
    const uint32_t kbuf = FP8 ? work_u32 : my_smem_u32 + (j % kDecStages) * kDecStageBytes;
    const uint32_t vbuf = kbuf + kSub * kD * 2;
    // ---- S = Q K^T : two 8-key n-tiles x 8 k-steps ------------------------------------------
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {        // 32 d per ldmatrix.x4
        uint32_t bfr[4];
        int r = nt * 8 + (lane & 7);
        int c = kk * 4 + (lane >> 3);
        ldmatrix_x4(bfr, kbuf + swz(r, c));
        mma16816<BF16>(s[nt], qa0[kk * 2], 0u, qa2[kk * 2], 0u, bfr[0], bfr[1]);
        mma16816<BF16>(s[nt], qa0[kk * 2 + 1], 0u, qa2[kk * 2 + 1], 0u, bfr[2], bfr[3]);
      }
    }
    // ---- scale, mask the tail, dump logits ----------------------------------------------------
    const int key0 = (st_begin + warp + j * kDecWarps) * kSub;
    float tmax = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        int key = key0 + nt * 8 + quad * 2 + e;
        float x = s[nt][e] * p.scale2;
        if (FP8) x *= __shfl_sync(0xFFFFFFFFu, sk0, nt * 8 + quad * 2 + e);    // the key's own scale
        x = key < n ? x : -INFINITY;
        s[nt][e] = x;
        tmax = fmaxf(tmax, x);
      }
      if (WRITE_LOGITS && row_head < kHg) {
        int key = key0 + nt * 8 + quad * 2;
        float* lp = p.logits + ((int64_t)b * p.H + g * kHg + row_head) * p.logit_stride + key;
        if (key + 1 < n) {
          *reinterpret_cast<float2*>(lp) = make_float2(s[nt][0], s[nt][1]);
        } else if (key < n) {
          lp[0] = s[nt][0];
        }
      }
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 2));
    const float m_new = fmaxf(m_run, tmax);       // finite: every sub-tile has >= 1 valid key
    const float alpha = exp2f(m_run - m_new);
    float psum = 0.f;
    uint32_t pa0, pa2;
    {
      float p00 = exp2f(s[0][0] - m_new), p01 = exp2f(s[0][1] - m_new);
      float p10 = exp2f(s[1][0] - m_new), p11 = exp2f(s[1][1] - m_new);
      psum = p00 + p01 + p10 + p11;
      if (FP8 && HAS_V) {                       // P.V sees the stored values: the rows' scales go on the probabilities
        p00 *= __shfl_sync(0xFFFFFFFFu, sv0, quad * 2);
        p01 *= __shfl_sync(0xFFFFFFFFu, sv0, quad * 2 + 1);
        p10 *= __shfl_sync(0xFFFFFFFFu, sv0, 8 + quad * 2);
        p11 *= __shfl_sync(0xFFFFFFFFu, sv0, 8 + quad * 2 + 1);
      }
      pa0 = pack_half2<BF16>(p00, p01);
      pa2 = pack_half2<BF16>(p10, p11);
    }
    psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 1);
    psum += __shfl_xor_sync(0xFFFFFFFFu, psum, 2);
    l_run = l_run * alpha + psum;
    m_run = m_new;
    if (HAS_V) {
      if (row_head >= kHg) { pa0 = 0u; pa2 = 0u; }
      // ---- O = O*alpha + P V : 16 d-tiles of 8 -------------------------------------------------
#pragma unroll
      for (int dt = 0; dt < 8; ++dt) {            // two 8-wide d tiles per ldmatrix.x4.trans
        uint32_t bfr[4];
        int r = (lane & 7) + ((lane >> 3) & 1) * 8;   // matrices: (k0-7,d0) (k8-15,d0) (k0-7,d1) (k8-15,d1)
        int c = dt * 2 + (lane >> 4);
        ldmatrix_x4_trans(bfr, vbuf + swz(r, c));
#pragma unroll
        for (int e = 0; e < 4; ++e) { o_acc[dt * 2][e] *= alpha; o_acc[dt * 2 + 1][e] *= alpha; }
        mma16816<BF16>(o_acc[dt * 2], pa0, 0u, pa2, 0u, bfr[0], bfr[1]);
        mma16816<BF16>(o_acc[dt * 2 + 1], pa0, 0u, pa2, 0u, bfr[2], bfr[3]);
      }
    }
    if (FP8) { sk0 = sk1; sv0 = sv1; sk1 = sk2; sv1 = sv2; }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the warps of this CTA through shared memory ------------------------------------------
  float* sm_m = reinterpret_cast<float*>(smem);                  // [warps][4]
  float* sm_l = sm_m + kDecWarps * kHg;                          // [warps][4]
  float* sm_o = sm_l + kDecWarps * kHg;                          // [warps][4][128]
  if (row_head < kHg) {
    if (quad == 0) { sm_m[warp * kHg + row_head] = m_run; sm_l[warp * kHg + row_head] = l_run; }
    if (HAS_V) {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        float* dst = sm_o + (warp * kHg + row_head) * kD + nt * 8 + quad * 2;
        dst[0] = o_acc[nt][0];
        dst[1] = o_acc[nt][1];
      }
    }
  }
  __syncthreads();
  for (int t = threadIdx.x; t < kHg * kD; t += blockDim.x) {
    const int h = t / kD, d = t % kD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm_m[w * kHg + h]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
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

static int default_splits(int batch, int G, int max_keys) {
  int64_t ctas = (int64_t)batch * G;
  if (ctas <= 0) return 1;
  int want = (int)((4LL * sm_count() + ctas - 1) / ctas);
  int cap = max_keys / 512;
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
  if (p.fp8) decode_attn_kernel<false, true, false, 2><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else if (p.bf16) decode_attn_kernel<false, true, false, 1><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else decode_attn_kernel<false, true, false, 0><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
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
  if (has_v && p.fp8) decode_attn_kernel<true, true, true, 2><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else if (has_v && p.bf16) decode_attn_kernel<true, true, true, 1><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else if (has_v) decode_attn_kernel<true, true, true, 0><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else if (p.fp8) decode_attn_kernel<true, false, true, 2><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else if (p.bf16) decode_attn_kernel<true, false, true, 1><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else decode_attn_kernel<true, false, true, 0><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
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
  if (p.fp8) decode_attn_kernel<false, true, false, 2><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else if (p.bf16) decode_attn_kernel<false, true, false, 1><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
  else decode_attn_kernel<false, true, false, 0><<<grid, kDecWarps * 32, kDecSmem, st>>>(p);
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
