// Memory-bound per-token kernels of the decoder step: residual-add + RMSNorm / LayerNorm, RoPE fused with
// the paged KV-cache write, gated activation, embedding gather, greedy argmax with log-prob, and the
// device-side bookkeeping that advances a decode batch by one token.
//
// Reference counterparts: `dropout_add_ln_fwd` (call site server/lorax_server/layers/layernorm.py:144-164),
// `rotary_emb.apply_rotary` (utils/layers.py:627-633), `reshape_and_cache` (utils/paged_attention.py:29-51),
// the eager `silu(gate) * up` (custom_modeling/flash_mistral_modeling.py:436-439) and the Triton metadata
// kernels (models/metadata_kernels.py:154-329).
#include <cuda_fp8.h>

#include "common.cuh"

namespace lx {

// ------------------------------------------------------------------------------------------------
// residual add + RMSNorm (or LayerNorm).  One CTA per token row, 16-byte loads, row kept in registers.
//   h = x (+ residual);  residual_out = h;  out = norm(h) * (w + w_offset) (+ b)
// ------------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;   // 256 threads * 8 vec * 8 elems = 16384 columns max

template <bool LAYERNORM>
__global__ void __launch_bounds__(kNormThreads)
norm_residual_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                     __nv_bfloat16* __restrict__ out, int H, long long ldx, long long ldr, long long ldo, float eps,
                     float w_offset, float x_scale) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int row = blockIdx.x;
  const int nvec = H / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * ldr) : nullptr;
  float vals[kNormMaxVec][8];
  float sum = 0.f, sumsq = 0.f;
#pragma unroll
  for (int it = 0; it < kNormMaxVec; ++it) {
    const int v = threadIdx.x + it * kNormThreads;
    if (v < nvec) {
      uint4 a = xr[v];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      float f[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 t = unpack_bf16x2(aw[q]);
        f[2 * q] = t.x * x_scale;
        f[2 * q + 1] = t.y * x_scale;
      }
      if (rr) {
        uint4 r = rr[v];
        const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 t = unpack_bf16x2(rw[q]);
          f[2 * q] += t.x;
          f[2 * q + 1] += t.y;
        }
        uint4 o;
        // the residual stream is stored in bf16; normalise the rounded value so both consumers agree
        o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
        o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
        rr[v] = o;
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 t = unpack_bf16x2(ow[q]);
          f[2 * q] = t.x;
          f[2 * q + 1] = t.y;
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        vals[it][q] = f[q];
        sum += f[q];
        sumsq += f[q] * f[q];
      }
    }
  }
  __shared__ float red[2][kNormThreads / 32];
  sum = warp_sum(sum);
  sumsq = warp_sum(sumsq);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = sum;
    red[1][threadIdx.x >> 5] = sumsq;
  }
  __syncthreads();
  float tsum = 0.f, tsq = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) {
    tsum += red[0][i];
    tsq += red[1][i];
  }
  float mean = 0.f, rstd;
  if (LAYERNORM) {
    mean = tsum / H;
    rstd = rsqrtf(fmaxf(tsq / H - mean * mean, 0.f) + eps);
  } else {
    rstd = rsqrtf(tsq / H + eps);
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = b ? reinterpret_cast<const uint4*>(b) : nullptr;
  uint4* orow = reinterpret_cast<uint4*>(out + row * ldo);
#pragma unroll
  for (int it = 0; it < kNormMaxVec; ++it) {
    const int v = threadIdx.x + it * kNormThreads;
    if (v < nvec) {
      uint4 ww = wr[v];
      const uint32_t wwv[4] = {ww.x, ww.y, ww.z, ww.w};
      uint32_t bwv[4] = {0, 0, 0, 0};
      if (br) {
        uint4 bb = br[v];
        bwv[0] = bb.x; bwv[1] = bb.y; bwv[2] = bb.z; bwv[3] = bb.w;
      }
      uint32_t ov[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 wf = unpack_bf16x2(wwv[q]);
        float2 bf = unpack_bf16x2(bwv[q]);
        float a0 = (vals[it][2 * q] - mean) * rstd * (wf.x + w_offset) + bf.x;
        float a1 = (vals[it][2 * q + 1] - mean) * rstd * (wf.y + w_offset) + bf.y;
        ov[q] = pack_bf16x2(a0, a1);
      }
      orow[v] = make_uint4(ov[0], ov[1], ov[2], ov[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE (rotate-half convention) on q and k in place, then scatter k and v into the paged cache.
//   qkv        [T, (nh + 2 nkv) * d]
//   cos_sin    [max_pos, rot] fp32: cos in [0, rot/2), sin in [rot/2, rot)
//   kv cache   [num_blocks, nkv, 2, page, d]   (K plane then V plane per (block, head))
//   slots      [T] flat slot index = block * page + offset; negative = do not cache
// One CTA per token; each thread rotates 4 pairs (8-byte loads).
// ------------------------------------------------------------------------------------------------
// Four bf16 (two packed words) times `inv_scale` as four e4m3 bytes, saturating.
LX_DEVICE uint32_t bf16x4_to_e4m3x4(uint2 w, float inv_scale) {
  const float2 a = unpack_bf16x2(w.x), b = unpack_bf16x2(w.y);
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv_scale, a.y * inv_scale), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv_scale, b.y * inv_scale), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__global__ void __launch_bounds__(256)
rope_kvwrite_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ cos_sin,
                    __nv_bfloat16* __restrict__ kv_cache, const int* __restrict__ slots, int nh, int nkv, int d, int rot,
                    int page, long long ldq, int apply_rope, int kv_fp8, float k_inv_scale, float v_inv_scale) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slots ? slots[t] : -1;
  __nv_bfloat16* row = qkv + t * ldq;
  const int half = rot / 2;
  const int quads_per_head = half / 4;           // groups of 4 pairs
  const float* cs = cos_sin + (long long)pos * rot;
  const int rope_heads = nh + nkv;
  long long blk = 0;
  int off = 0;
  if (slot >= 0) {
    blk = slot / page;
    off = slot % page;
  }
  // rotate q and k heads
  for (int idx = threadIdx.x; idx < rope_heads * quads_per_head; idx += blockDim.x) {
    const int head = idx / quads_per_head;
    const int qd = (idx % quads_per_head) * 4;
    __nv_bfloat16* hp = row + head * d;
    uint2 lo = *reinterpret_cast<uint2*>(hp + qd);
    uint2 hi = *reinterpret_cast<uint2*>(hp + half + qd);
    if (apply_rope) {
      const float4 c = *reinterpret_cast<const float4*>(cs + qd);
      const float4 s = *reinterpret_cast<const float4*>(cs + half + qd);
      float2 l0 = unpack_bf16x2(lo.x), l1 = unpack_bf16x2(lo.y);
      float2 h0 = unpack_bf16x2(hi.x), h1 = unpack_bf16x2(hi.y);
      float o0 = l0.x * c.x - h0.x * s.x, o1 = l0.y * c.y - h0.y * s.y;
      float o2 = l1.x * c.z - h1.x * s.z, o3 = l1.y * c.w - h1.y * s.w;
      float p0 = h0.x * c.x + l0.x * s.x, p1 = h0.y * c.y + l0.y * s.y;
      float p2 = h1.x * c.z + l1.x * s.z, p3 = h1.y * c.w + l1.y * s.w;
      lo = make_uint2(pack_bf16x2(o0, o1), pack_bf16x2(o2, o3));
      hi = make_uint2(pack_bf16x2(p0, p1), pack_bf16x2(p2, p3));
      *reinterpret_cast<uint2*>(hp + qd) = lo;
      *reinterpret_cast<uint2*>(hp + half + qd) = hi;
    }
    if (head >= nh && slot >= 0) {
      const int kh = head - nh;
      const long long e0 = (((blk * nkv + kh) * 2 + 0) * page + off) * d;
      if (kv_fp8) {
        // e4m3 cache: value / scale, saturating; 4 bytes per store
        uint8_t* dst = reinterpret_cast<uint8_t*>(kv_cache) + e0;
        *reinterpret_cast<uint32_t*>(dst + qd) = bf16x4_to_e4m3x4(lo, k_inv_scale);
        *reinterpret_cast<uint32_t*>(dst + half + qd) = bf16x4_to_e4m3x4(hi, k_inv_scale);
      } else {
        __nv_bfloat16* dst = kv_cache + e0;
        *reinterpret_cast<uint2*>(dst + qd) = lo;
        *reinterpret_cast<uint2*>(dst + half + qd) = hi;
      }
    }
  }
  if (slot >= 0) {
    // un-rotated tail of k (partial rotary) and the whole of v
    const int tail = d - rot;
    if (tail > 0) {
      for (int idx = threadIdx.x; idx < nkv * tail; idx += blockDim.x) {
        const int kh = idx / tail, e = rot + idx % tail;
        const long long at = (((blk * nkv + kh) * 2 + 0) * page + off) * d + e;
        if (kv_fp8) {
          reinterpret_cast<uint8_t*>(kv_cache)[at] =
              (uint8_t)__nv_cvt_float_to_fp8(__bfloat162float(row[(nh + kh) * d + e]) * k_inv_scale, __NV_SATFINITE, __NV_E4M3);
        } else {
          kv_cache[at] = row[(nh + kh) * d + e];
        }
      }
    }
    const int vec_per_head = d / 8;
    for (int idx = threadIdx.x; idx < nkv * vec_per_head; idx += blockDim.x) {
      const int kh = idx / vec_per_head, e = (idx % vec_per_head) * 8;
      const uint4 v = *reinterpret_cast<const uint4*>(row + (nh + nkv + kh) * d + e);
      const long long at = (((blk * nkv + kh) * 2 + 1) * page + off) * d + e;
      if (kv_fp8) {
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(kv_cache) + at) =
            make_uint2(bf16x4_to_e4m3x4(make_uint2(v.x, v.y), v_inv_scale), bf16x4_to_e4m3x4(make_uint2(v.z, v.w), v_inv_scale));
      } else {
        *reinterpret_cast<uint4*>(kv_cache + at) = v;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]
// ------------------------------------------------------------------------------------------------
enum Act : int { kSilu = 0, kGelu = 1, kGeluTanh = 2, kRelu = 3 };
template <int ACT>
LX_DEVICE float act_fn(float x) {
  if (ACT == kSilu) return x / (1.f + __expf(-x));
  if (ACT == kGelu) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  if (ACT == kGeluTanh) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return fmaxf(x, 0.f);
}
template <int ACT, bool GATED>
__global__ void __launch_bounds__(256)
act_mul_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int I, long long ldi, long long ldo, long long total_vec) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int vec_per_row = I / 8;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total_vec; v += (long long)gridDim.x * blockDim.x) {
    const long long t = v / vec_per_row;
    const int c = (int)(v % vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(in + t * ldi + c);
    uint4 u = make_uint4(0, 0, 0, 0);
    if (GATED) u = *reinterpret_cast<const uint4*>(in + t * ldi + I + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 a = unpack_bf16x2(gw[q]);
      float r0 = act_fn<ACT>(a.x), r1 = act_fn<ACT>(a.y);
      if (GATED) {
        float2 b = unpack_bf16x2(uw[q]);
        r0 *= b.x;
        r1 *= b.y;
      }
      ow[q] = pack_bf16x2(r0, r1);
    }
    *reinterpret_cast<uint4*>(out + t * ldo + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding gather with vocabulary range [v0, v1): rows outside are written as zero (vocab-parallel).
struct EmbedPeerParams {
  const __nv_bfloat16* tables[8];     // every rank's shard, as mapped into this process
  int rows_per_rank, world, vocab, H;
  float mult;
};

__global__ void __launch_bounds__(128) embed_peer_kernel(const int* __restrict__ ids, const EmbedPeerParams p, __nv_bfloat16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int t = blockIdx.x;
  const int id = ids[t];
  uint4* o = reinterpret_cast<uint4*>(out + (long long)t * p.H);
  const int owner = id >= 0 ? id / p.rows_per_rank : p.world;
  if (id < 0 || id >= p.vocab || owner >= p.world) {
    for (int v = threadIdx.x; v < p.H / 8; v += blockDim.x) o[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(p.tables[owner] + (long long)(id - owner * p.rows_per_rank) * p.H);
  for (int v = threadIdx.x; v < p.H / 8; v += blockDim.x) {
    uint4 a = src[v];
    if (p.mult != 1.f) {
      uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = unpack_bf16x2(w[q]);
        w[q] = pack_bf16x2(f.x * p.mult, f.y * p.mult);
      }
      a = make_uint4(w[0], w[1], w[2], w[3]);
    }
    o[v] = a;
  }
}

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, __nv_bfloat16* __restrict__ out, int H,
             int v0, int v1, float mult) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int t = blockIdx.x;
  const int id = ids[t];
  uint4* o = reinterpret_cast<uint4*>(out + (long long)t * H);
  if (id < v0 || id >= v1) {
    for (int v = threadIdx.x; v < H / 8; v += blockDim.x) o[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (long long)(id - v0) * H);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    uint4 a = src[v];
    if (mult != 1.f) {
      uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = unpack_bf16x2(w[q]);
        w[q] = pack_bf16x2(f.x * mult, f.y * mult);
      }
      a = make_uint4(w[0], w[1], w[2], w[3]);
    }
    o[v] = a;
  }
}

// ------------------------------------------------------------------------------------------------
// Greedy head: per row argmax and log-softmax value of the argmax over bf16 logits [T, V].
// Lowest index wins ties (matches torch.argmax on CPU for the oracle tests).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
argmax_logprob_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int V, int* __restrict__ ids,
                      float* __restrict__ logprobs, float softcap) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int t = blockIdx.x;
  const __nv_bfloat16* row = logits + t * ld;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  float m = -INFINITY, s = 0.f;   // online logsumexp
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float x = __bfloat162float(row[i]);
    if (softcap > 0.f) x = softcap * tanhf(x / softcap);
    if (x > best || (x == best && i < besti)) { best = x; besti = i; }
    if (x > m) { s = s * __expf(m - x) + 1.f; m = x; }
    else s += __expf(x - m);
  }
  __shared__ float sb[16], sm[16], ss[16];
  __shared__ int si[16];
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    float om = __shfl_xor_sync(0xffffffffu, m, o);
    float os = __shfl_xor_sync(0xffffffffu, s, o);
    if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { sb[w] = best; si[w] = besti; sm[w] = m; ss[w] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
      if (sb[i] > best || (sb[i] == best && si[i] < besti)) { best = sb[i]; besti = si[i]; }
      float nm = fmaxf(m, sm[i]);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (sm[i] == -INFINITY ? 0.f : ss[i] * __expf(sm[i] - nm));
      m = nm;
    }
    ids[t] = besti;
    if (logprobs) logprobs[t] = best - (m + __logf(s));
  }
}

// ------------------------------------------------------------------------------------------------
// Advance a decode batch by one token entirely on the device (no host round trip between graph replays):
//   input_ids <- next_ids; positions += 1; ctx_lens += 1; slots from the block table.
// A row with ctx_lens < 0 is padding and is left alone.
// ------------------------------------------------------------------------------------------------
__global__ void advance_decode_kernel(int* __restrict__ input_ids, const int* __restrict__ next_ids, int* __restrict__ positions,
                                      int* __restrict__ ctx_lens, int* __restrict__ slots, const int* __restrict__ block_tables,
                                      int max_blocks, int page, int B) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  if (ctx_lens[b] <= 0) { slots[b] = -1; return; }
  input_ids[b] = next_ids[b];
  const int pos = positions[b] + 1;
  positions[b] = pos;
  ctx_lens[b] = pos + 1;
  const int blk = block_tables[(long long)b * max_blocks + pos / page];
  slots[b] = blk * page + pos % page;
}

__global__ void __launch_bounds__(256)
prefill_metadata_kernel(const int* __restrict__ cu_q, const int* __restrict__ cache_lens, const int* __restrict__ seq_slot,
                        const int* __restrict__ block_tables, int max_blocks, int B, int page, int T, int* __restrict__ positions,
                        int* __restrict__ slots, int* __restrict__ tok_slot) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  int lo = 0, hi = B;                     // last sequence whose first token is at or before t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid;
  }
  const int pos = cache_lens[lo] + (t - cu_q[lo]);
  positions[t] = pos;
  const int blk = min(pos / page, max_blocks - 1);
  slots[t] = block_tables[(long long)lo * max_blocks + blk] * page + pos % page;
  if (tok_slot != nullptr) tok_slot[t] = seq_slot[lo];
}

}  // namespace lx

extern "C" {

int lx_norm_residual(const void* x, void* residual, const void* w, const void* b, void* out, int T, int H, long long ldx,
                     long long ldr, long long ldo, float eps, float w_offset, float x_scale, int layernorm, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (H % 8 != 0 || H > kNormThreads * kNormMaxVec * 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<__nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto Bv = reinterpret_cast<const __nv_bfloat16*>(b);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  if (layernorm) launch_pdl(norm_residual_kernel<true>, dim3(T), dim3(kNormThreads), 0, s, X, R, W, Bv, O, H, ldx, ldr, ldo, eps, w_offset, x_scale);
  else launch_pdl(norm_residual_kernel<false>, dim3(T), dim3(kNormThreads), 0, s, X, R, W, Bv, O, H, ldx, ldr, ldo, eps, w_offset, x_scale);
  return -(int)cudaGetLastError();
}

// kv_fp8 != 0: the cache holds e4m3 bytes, value / k_scale for keys and value / v_scale for values (same layout).
int lx_rope_kvwrite_kv8(void* qkv, const int* positions, const float* cos_sin, void* kv_cache, const int* slots, int T, int nh,
                        int nkv, int d, int rot, int page, long long ldq, int apply_rope, int kv_fp8, float k_scale, float v_scale,
                        void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (d % 8 != 0 || rot % 8 != 0 || rot > d) return -1;
  if (kv_fp8 && (k_scale <= 0.f || v_scale <= 0.f)) return -2;
  launch_pdl(rope_kvwrite_kernel, dim3(T), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<__nv_bfloat16*>(qkv), positions, cos_sin, reinterpret_cast<__nv_bfloat16*>(kv_cache), slots, nh, nkv, d,
      rot, page, ldq, apply_rope, kv_fp8, kv_fp8 ? 1.f / k_scale : 1.f, kv_fp8 ? 1.f / v_scale : 1.f);
  return -(int)cudaGetLastError();
}

int lx_rope_kvwrite(void* qkv, const int* positions, const float* cos_sin, void* kv_cache, const int* slots, int T, int nh,
                    int nkv, int d, int rot, int page, long long ldq, int apply_rope, void* stream) {
  return lx_rope_kvwrite_kv8(qkv, positions, cos_sin, kv_cache, slots, T, nh, nkv, d, rot, page, ldq, apply_rope, 0, 1.f, 1.f, stream);
}

int lx_act_mul(const void* in, void* out, int T, int I, long long ldi, long long ldo, int act, int gated, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (I % 8 != 0) return -1;
  const long long total = (long long)T * (I / 8);
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(in);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
#define LX_ACT(A)                                                                         \
  if (gated) launch_pdl(act_mul_kernel<A, true>, dim3(grid), dim3(256), 0, s, X, O, I, ldi, ldo, total);      \
  else launch_pdl(act_mul_kernel<A, false>, dim3(grid), dim3(256), 0, s, X, O, I, ldi, ldo, total);
  switch (act) {
    case kSilu: LX_ACT(kSilu); break;
    case kGelu: LX_ACT(kGelu); break;
    case kGeluTanh: LX_ACT(kGeluTanh); break;
    default: LX_ACT(kRelu); break;
  }
#undef LX_ACT
  return -(int)cudaGetLastError();
}

int lx_embed(const int* ids, const void* table, void* out, int T, int H, int v0, int v1, float mult, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  launch_pdl(embed_kernel, dim3(T), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), ids, reinterpret_cast<const __nv_bfloat16*>(table),
                                                                      reinterpret_cast<__nv_bfloat16*>(out), H, v0, v1, mult);
  return -(int)cudaGetLastError();
}

// Vocabulary-parallel embedding without a collective: rank r owns rows [r * rows_per_rank, (r + 1) * rows_per_rank) of the
// table in peer-mapped memory and every rank reads the rows it needs straight from the owner over NVLink (plain peer loads of
// a table that never changes: nothing to wait for).  Replaces embedding lookup + all-reduce of [T, H]
// (server/lorax_server/layers/tensor_parallel.py:153-190 masks out-of-shard ids and all-reduces).
int lx_embed_peer(const int* ids, const void* peer_tables, void* out, int T, int H, int rows_per_rank, int world, int vocab, float mult,
                  void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (H % 8 != 0 || world < 1 || world > 8) return -1;
  EmbedPeerParams p{};
  const unsigned long long* tabs = reinterpret_cast<const unsigned long long*>(peer_tables);
  for (int r = 0; r < world; ++r) p.tables[r] = reinterpret_cast<const __nv_bfloat16*>(tabs[r]);
  p.rows_per_rank = rows_per_rank; p.world = world; p.vocab = vocab; p.H = H; p.mult = mult;
  launch_pdl(embed_peer_kernel, dim3(T), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), ids, p, reinterpret_cast<__nv_bfloat16*>(out));
  return -(int)cudaGetLastError();
}

int lx_argmax_logprob(const void* logits, long long ld, int T, int V, int* ids, float* logprobs, float softcap, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  launch_pdl(argmax_logprob_kernel, dim3(T), dim3(512), 0, reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(logits), ld, V,
                                                                             ids, logprobs, softcap);
  return -(int)cudaGetLastError();
}

// Per-token metadata of a ragged prefill from its per-sequence description: positions[t] = cache_lens[b] + (t - cu_q[b]),
// slots[t] = block_tables[b][position / page] * page + position % page, tok_slot[t] = seq_slot[b], for the sequence b that
// holds token t (binary search in cu_q).  The reference assembles these arrays on the host for every batch
// (server/lorax_server/models/flash_causal_lm.py:200-420).
int lx_prefill_metadata(const int* cu_q, const int* cache_lens, const int* seq_slot, const int* block_tables, int max_blocks, int B,
                        int page, int T, int* positions, int* slots, int* tok_slot, void* stream) {
  using namespace lx;
  if (T <= 0 || B <= 0) return 0;
  launch_pdl(prefill_metadata_kernel, dim3((T + 255) / 256), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), cu_q, cache_lens, seq_slot,
             block_tables, max_blocks, B, page, T, positions, slots, tok_slot);
  return -(int)cudaGetLastError();
}

int lx_advance_decode(int* input_ids, const int* next_ids, int* positions, int* ctx_lens, int* slots, const int* block_tables,
                      int max_blocks, int page, int B, void* stream) {
  using namespace lx;
  if (B <= 0) return 0;
  launch_pdl(advance_decode_kernel, dim3((B + 127) / 128), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), input_ids, next_ids, positions, ctx_lens,
                                                                                          slots, block_tables, max_blocks, page, B);
  return -(int)cudaGetLastError();
}

}  // extern "C"
