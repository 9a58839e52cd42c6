// KV-cache write path: optional per-head RMS norm of Q and K (Qwen3), rotary position embedding of Q
// and K (the half-rotation convention of the Hugging Face Llama / Qwen3 models), and the append of the
// new K / V rows into the paged (or contiguous) cache — one pass over the new tokens, so that the
// attention kernels find the cache in the layout they read, without the transposes and
// `.contiguous()` copies the reference's strategy pays before every kernel call
// (strategies/EfficientKascadeStrategy.py:144-150).  Bound by HBM: each new row is read once and
// written once.
//
// Arithmetic follows the Hugging Face modules step by step, in the model's type (fp16 or bf16), so that
// results agree to the last bit wherever sin / cos round the same way: the norm is computed in fp32 and
// rounded to that type before the gain is applied (LlamaRMSNorm / Qwen3RMSNorm), cos and sin are computed
// in fp32 from position * inv_freq[i] (the model's own inverse-frequency table, so every rope-scaling
// variant is covered), scaled and rounded to that type, and  x * cos + rotate_half(x) * sin  is evaluated
// in that type with a rounding after each product and after the sum (apply_rotary_pos_emb).
#include <cuda_bf16.h>

#include "common.cuh"

namespace kb200 {

struct KvWriteParams {
  const __half* q_in; __half* q_out; int64_t q_sb, q_st, q_sh;      // [B, T, H, D] views (q_out contiguous)
  const __half* k_new; int64_t k_sb, k_st, k_sh;                     // [B, T, G, D]
  const __half* v_new; int64_t v_sb, v_st, v_sh;
  const int32_t* start_pos;                                           // [B] cache length before the append
  const int32_t* n_new;                                               // [B] or null (= T)
  __half* k_cache; __half* v_cache;
  int64_t c_sb, c_sp, c_st, c_sh;                                     // cache strides (batch, page, token, head)
  const int32_t* block_table; int bt_stride; int page_shift, page_mask;
  const __half* q_gain; const __half* k_gain; float eps;              // RMS-norm gains [D] or null
  // FP8 (e4m3) cache: a row is stored as value / scale of its (page, KV head); strides of the cache in bytes
  const float* k_scale; const float* v_scale; int64_t s_sb, s_sp, s_sh;
  const float* inv_freq; float rope_scale;                            // [D/2] inverse frequencies or null (no rotary)
  int B, T, H, G;
};

// One CTA per (sequence, new token): the token's 64 (cos, sin) pairs are computed once and shared by all
// its heads; a row of 128 values is handled by 8 lanes (lane c holds elements 8c..8c+7 and
// 64+8c..64+8c+7: the two elements a rotation pairs up sit in the same lane, 16-byte loads and stores),
// a warp takes four rows at a time.
constexpr int kKvWriteThreads = 192;

// The storage type of the activations and the cache: fp16, or bf16 (the pointers of KvWriteParams are then
// bf16 in disguise).  Every rounding step is the one the Hugging Face modules take in that type.
template <bool BF16> struct Pair { using T = __half2; using S = __half; };
template <> struct Pair<true> { using T = __nv_bfloat162; using S = __nv_bfloat16; };
__device__ __forceinline__ float2 to_f2(__half2 x) { return __half22float2(x); }
__device__ __forceinline__ float2 to_f2(__nv_bfloat162 x) { return __bfloat1622float2(x); }
template <bool BF16> __device__ __forceinline__ typename Pair<BF16>::T from_f2(float a, float b) {
  if constexpr (BF16) return __floats2bfloat162_rn(a, b);
  else return __floats2half2_rn(a, b);
}
template <bool BF16> __device__ __forceinline__ typename Pair<BF16>::S from_f(float a) {
  if constexpr (BF16) return __float2bfloat16_rn(a);
  else return __float2half_rn(a);
}

// eight values of the storage type (four pairs) -> eight e4m3 bytes of value / scale (fp32 division, saturating,
// round to nearest even)
template <typename H2>
__device__ __forceinline__ uint2 quantize8(const H2* x, float scale) {
  uint32_t w[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 a = to_f2(x[2 * i]), b = to_f2(x[2 * i + 1]);
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(lo) : "f"(a.y / scale), "f"(a.x / scale));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(hi) : "f"(b.y / scale), "f"(b.x / scale));
    w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

template <bool BF16, bool FP8>
__global__ void __launch_bounds__(kKvWriteThreads) kv_write_kernel(const KvWriteParams p) {
  using H2 = typename Pair<BF16>::T;
  using H1 = typename Pair<BF16>::S;
  __shared__ __align__(16) H1 cos_s[kD / 2];
  __shared__ __align__(16) H1 sin_s[kD / 2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x / p.T, t = blockIdx.x - b * p.T;
  const int n = p.n_new ? p.n_new[b] : p.T;
  if (t >= n) return;
  const int pos = p.start_pos[b] + t;
  if (p.inv_freq && tid < kD / 2) {
    float sn, cs;
    sincosf((float)pos * p.inv_freq[tid], &sn, &cs);
    cos_s[tid] = from_f<BF16>(cs * p.rope_scale);
    sin_s[tid] = from_f<BF16>(sn * p.rope_scale);
  }
  __syncthreads();
  const int heads = p.H + 2 * p.G;                                   // Q heads, K heads, V heads
  const int c = lane & 7;
  for (int h0 = warp * 4; h0 < heads; h0 += (kKvWriteThreads / 32) * 4) {   // uniform per warp
    const int h = min(h0 + (lane >> 3), heads - 1);
    const bool active = h0 + (lane >> 3) < heads;                    // the last group of rows may be partial
    const int kind = h < p.H ? 0 : (h < p.H + p.G ? 1 : 2);          // 0 = Q, 1 = K, 2 = V
    const int hh = kind == 0 ? h : (kind == 1 ? h - p.H : h - p.H - p.G);
    const __half* src = kind == 0 ? p.q_in + b * p.q_sb + t * p.q_st + hh * p.q_sh
                      : kind == 1 ? p.k_new + b * p.k_sb + t * p.k_st + hh * p.k_sh
                                  : p.v_new + b * p.v_sb + t * p.v_st + hh * p.v_sh;
    uint4 lo4 = reinterpret_cast<const uint4*>(src)[c];              // elements 8c .. 8c+7
    uint4 hi4 = reinterpret_cast<const uint4*>(src + kD / 2)[c];     // elements 64+8c .. 64+8c+7
    H2* lo = reinterpret_cast<H2*>(&lo4);
    H2* hi = reinterpret_cast<H2*>(&hi4);
    const __half* gain = kind == 0 ? p.q_gain : (kind == 1 ? p.k_gain : nullptr);
    // sum of squares of the row: all lanes of the warp take part in the shuffles, whatever their row is
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = to_f2(lo[e]), d2 = to_f2(hi[e]);
      ss += a.x * a.x + a.y * a.y + d2.x * d2.x + d2.y * d2.y;
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if (gain) {
      // x.float() * rsqrt(mean(x^2) + eps), rounded to the storage type, times the gain (a product in that type)
      const float r = rsqrtf(ss / kD + p.eps);
      const uint4 g_lo4 = reinterpret_cast<const uint4*>(gain)[c];
      const uint4 g_hi4 = reinterpret_cast<const uint4*>(gain + kD / 2)[c];
      const H2* g_lo = reinterpret_cast<const H2*>(&g_lo4);
      const H2* g_hi = reinterpret_cast<const H2*>(&g_hi4);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = to_f2(lo[e]), d2 = to_f2(hi[e]);
        lo[e] = __hmul2_rn(g_lo[e], from_f2<BF16>(a.x * r, a.y * r));
        hi[e] = __hmul2_rn(g_hi[e], from_f2<BF16>(d2.x * r, d2.y * r));
      }
    }
    if (kind != 2 && p.inv_freq) {
      const uint4 cs4 = reinterpret_cast<const uint4*>(cos_s)[c];
      const uint4 sn4 = reinterpret_cast<const uint4*>(sin_s)[c];
      const H2* cs = reinterpret_cast<const H2*>(&cs4);
      const H2* sn = reinterpret_cast<const H2*>(&sn4);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // first half:  x_lo * cos + (-x_hi) * sin ; second half:  x_hi * cos + x_lo * sin
        // (the _rn forms are never contracted into a fused multiply-add, which would skip a rounding)
        const H2 new_lo = __hadd2_rn(__hmul2_rn(lo[e], cs[e]), __hmul2_rn(__hneg2(hi[e]), sn[e]));
        const H2 new_hi = __hadd2_rn(__hmul2_rn(hi[e], cs[e]), __hmul2_rn(lo[e], sn[e]));
        lo[e] = new_lo;
        hi[e] = new_hi;
      }
    }
    __half* dst;
    if (kind == 0) {
      dst = p.q_out + (((int64_t)b * p.T + t) * p.H + hh) * kD;
    } else {
      const int page = pos >> p.page_shift, slot = pos & p.page_mask;
      const int64_t phys = p.block_table ? (int64_t)p.block_table[(int64_t)b * p.bt_stride + page] : page;
      if (FP8) {
        if (active) {
          const float sc = (kind == 1 ? p.k_scale : p.v_scale)[b * p.s_sb + phys * p.s_sp + hh * p.s_sh];
          uint8_t* d8 = reinterpret_cast<uint8_t*>(kind == 1 ? p.k_cache : p.v_cache) + b * p.c_sb + phys * p.c_sp +
                        slot * p.c_st + hh * p.c_sh;
          reinterpret_cast<uint2*>(d8)[c] = quantize8(lo, sc);              // bytes 8c .. 8c+7
          reinterpret_cast<uint2*>(d8 + kD / 2)[c] = quantize8(hi, sc);     // bytes 64+8c .. 64+8c+7
        }
        continue;
      }
      dst = (kind == 1 ? p.k_cache : p.v_cache) + b * p.c_sb + phys * p.c_sp + slot * p.c_st + hh * p.c_sh;
    }
    if (active) {
      reinterpret_cast<uint4*>(dst)[c] = lo4;
      reinterpret_cast<uint4*>(dst + kD / 2)[c] = hi4;
    }
  }
}

}  // namespace kb200

extern "C" int kb200_kv_write(const kb200_act_layout* q_in, void* q_out, const kb200_act_layout* k_new,
                              const kb200_act_layout* v_new, const int32_t* start_pos, const int32_t* n_new,
                              const kb200_kv_layout* kv, const void* q_norm_gain, const void* k_norm_gain,
                              float norm_eps, const float* inv_freq, float rope_scale, int batch, int max_new,
                              int num_q_heads, int num_kv_heads, void* stream) {
  using namespace kb200;
  KB_ENTRY(k_new ? k_new->ptr : nullptr, "kv_write: k_new");
  KB_REQUIRE(k_new && k_new->ptr && v_new && v_new->ptr && start_pos && kv && kv->k && kv->v,
             "kv_write: null pointer");
  KB_REQUIRE(batch >= 0 && max_new >= 0 && num_kv_heads > 0 && num_q_heads >= 0, "kv_write: bad sizes");
  const bool fp8 = kv->dtype == KB200_FP8_E4M3;
  KB_REQUIRE((k_new->dtype == KB200_FP16 || k_new->dtype == KB200_BF16) && v_new->dtype == k_new->dtype &&
                 (fp8 || kv->dtype == k_new->dtype) && (!q_in || !q_in->ptr || q_in->dtype == k_new->dtype),
             "kv_write: q / k / v and the cache must all be fp16 or all bf16 (its arithmetic follows the Hugging Face "
             "modules step by step in that type; gains are in the same type), or the cache FP8 (e4m3) with scales");
  KB_REQUIRE(!fp8 || (kv->k_scale && kv->v_scale), "kv_write: an FP8 cache needs k_scale / v_scale");
  const bool bf16 = k_new->dtype == KB200_BF16;
  KB_REQUIRE(kv->page_size >= 1 && (kv->page_size & (kv->page_size - 1)) == 0,
             "kv_write: page_size must be a power of two (got %d)", kv->page_size);
  KB_REQUIRE(!inv_freq || (reinterpret_cast<uintptr_t>(inv_freq) & 7) == 0, "kv_write: inv_freq must be 8-byte aligned");
  const bool with_q = q_in && q_in->ptr;
  KB_REQUIRE(!with_q || q_out, "kv_write: q_in given without q_out");
  auto aligned = [](const void* ptr, int64_t a, int64_t b2, int64_t c) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && a % 8 == 0 && b2 % 8 == 0 && c % 8 == 0;
  };
  KB_REQUIRE(aligned(k_new->ptr, k_new->stride_b, k_new->stride_t, k_new->stride_h) &&
                 aligned(v_new->ptr, v_new->stride_b, v_new->stride_t, v_new->stride_h) &&
                 (!with_q || aligned(q_in->ptr, q_in->stride_b, q_in->stride_t, q_in->stride_h)) &&
                 aligned(kv->k, kv->stride_batch, kv->stride_page, kv->stride_token) &&
                 aligned(kv->v, kv->stride_head, 0, 0),
             "kv_write: pointers must be 16-byte aligned and strides multiples of 8 elements");
  KB_REQUIRE(!fp8 || (kv->stride_batch % 16 == 0 && kv->stride_page % 16 == 0 && kv->stride_token % 16 == 0 &&
                      kv->stride_head % 16 == 0),
             "kv_write: strides of an FP8 cache must be multiples of 16 bytes");
  if (batch == 0 || max_new == 0) return 0;
  KvWriteParams p{};
  if (with_q) {
    p.q_in = static_cast<const __half*>(q_in->ptr);
    p.q_sb = q_in->stride_b; p.q_st = q_in->stride_t; p.q_sh = q_in->stride_h;
    p.q_out = static_cast<__half*>(q_out);
  }
  p.k_new = static_cast<const __half*>(k_new->ptr);
  p.k_sb = k_new->stride_b; p.k_st = k_new->stride_t; p.k_sh = k_new->stride_h;
  p.v_new = static_cast<const __half*>(v_new->ptr);
  p.v_sb = v_new->stride_b; p.v_st = v_new->stride_t; p.v_sh = v_new->stride_h;
  p.start_pos = start_pos;
  p.n_new = n_new;
  p.k_cache = static_cast<__half*>(const_cast<void*>(kv->k));
  p.v_cache = static_cast<__half*>(const_cast<void*>(kv->v));
  p.c_sb = kv->stride_batch; p.c_sp = kv->stride_page; p.c_st = kv->stride_token; p.c_sh = kv->stride_head;
  p.block_table = kv->block_table;
  p.bt_stride = kv->block_table_stride;
  int shift = 0;
  while ((1 << shift) < kv->page_size) ++shift;
  p.page_shift = shift;
  p.page_mask = kv->page_size - 1;
  p.k_scale = kv->k_scale;
  p.v_scale = kv->v_scale;
  p.s_sb = kv->scale_stride_batch; p.s_sp = kv->scale_stride_page; p.s_sh = kv->scale_stride_head;
  p.q_gain = static_cast<const __half*>(q_norm_gain);
  p.k_gain = static_cast<const __half*>(k_norm_gain);
  p.eps = norm_eps;
  p.inv_freq = inv_freq;
  p.rope_scale = rope_scale;
  p.B = batch; p.T = max_new; p.H = with_q ? num_q_heads : 0; p.G = num_kv_heads;
  const int64_t blocks = (int64_t)batch * max_new;                   // one CTA per (sequence, new token)
  KB_REQUIRE(blocks < (1ll << 31), "kv_write: too many tokens for one launch");
  cudaStream_t st = (cudaStream_t)stream;
  if (bf16 && fp8) kv_write_kernel<true, true><<<(unsigned)blocks, kKvWriteThreads, 0, st>>>(p);
  else if (bf16) kv_write_kernel<true, false><<<(unsigned)blocks, kKvWriteThreads, 0, st>>>(p);
  else if (fp8) kv_write_kernel<false, true><<<(unsigned)blocks, kKvWriteThreads, 0, st>>>(p);
  else kv_write_kernel<false, false><<<(unsigned)blocks, kKvWriteThreads, 0, st>>>(p);
  KB_CHECK_LAUNCH("kv_write_kernel");
  return 0;
}
