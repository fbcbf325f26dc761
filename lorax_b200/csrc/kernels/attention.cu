// Attention over the paged KV cache.
//
//   attn_decode_kernel   one query token per row, GQA group packed into the MMA M dimension, keys split
//                        across the four warps of a CTA (each with a private cp.async pipeline) and
//                        optionally across CTAs (split-KV with a second combine pass).
//   attn_prefill_kernel  causal flash attention for ragged (padding-free) prompt chunks; K and V are read
//                        from the paged cache, so plain prefill, chunked prefill and prefill on top of a
//                        cached prefix are the same code path.
//
// Both honour a sliding window and logit soft-capping.  They stand in for the reference's third-party
// kernels: vLLM `paged_attention_v1/v2` (call site server/lorax_server/utils/paged_attention.py:127-178) and
// flash-attn `varlen_fwd` (utils/flash_attn.py:180-201).
//
// Cache layout (one tensor per layer): [num_blocks, kv_heads, 2, PAGE, D] -- for each (block, head) the K
// plane [PAGE, D] is followed by the V plane, so one page of one head is a single contiguous 2*PAGE*D run.
//
// fp8 cache (template flag KV8): pages hold e4m3 bytes in the same layout, written by `rope_kvwrite` as value / scale with one
// scale for K and one for V per layer (the reference's k_scale / v_scale, server/lorax_server/utils/paged_attention.py:23-47).
// A page arrives in shared memory as bytes (half the traffic of the bf16 cache, which is what bounds decode attention) and is
// expanded to a bf16 plane before the MMAs; the K scale is folded into the softmax scale and the V scale into the output.
#include <cuda_fp8.h>

#include "common.cuh"

namespace lx {

constexpr int kPage = 32;
constexpr float kLog2e = 1.4426950408889634f;

LX_DEVICE void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
LX_DEVICE void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
LX_DEVICE void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// A [ROWS, D] bf16 plane in shared memory; 16-byte chunk c of row r lives at chunk (c ^ (r & 7)) so that
// ldmatrix (8 rows, same logical chunk) touches 8 different bank groups.
template <int D>
LX_DEVICE uint32_t swz(int r, int c) { return (uint32_t)((r * (D / 8) + (c ^ (r & 7))) * 16); }

// Copy ROWS x D bf16 (contiguous in global memory) into a swizzled plane with `NT` cooperating threads.
template <int D, int ROWS, int NT>
LX_DEVICE void load_plane(uint32_t smem_base, const __nv_bfloat16* g, int tid, bool valid) {
  constexpr int CPR = D / 8;
  constexpr int CHUNKS = ROWS * CPR;
#pragma unroll
  for (int c = tid; c < CHUNKS; c += NT) {
    const int r = c / CPR, cc = c % CPR;
    const uint32_t dst = smem_base + swz<D>(r, cc);
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(g + (long long)c * 8), "r"(sz) : "memory");
  }
}

// Copy ROWS x D e4m3 bytes (contiguous in global memory) into a linear staging area.
template <int D, int ROWS, int NT>
LX_DEVICE void load_plane8(uint32_t smem_base, const uint8_t* g, int tid, bool valid) {
  constexpr int CHUNKS = ROWS * D / 16;
#pragma unroll
  for (int c = tid; c < CHUNKS; c += NT) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_base + c * 16), "l"(g + (long long)c * 16), "r"(sz) : "memory");
  }
}
LX_DEVICE uint32_t e4m3x2_to_bf16x2(uint32_t two) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(two & 0xffffu), __NV_E4M3);
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
  return pack_bf16x2(f.x, f.y);
}
// Expand a staged e4m3 plane into a swizzled bf16 plane (every e4m3 value is exact in bf16).
template <int D, int ROWS, int NT>
LX_DEVICE void expand_plane8(uint32_t dst_plane, uint32_t src8, int tid) {
  constexpr int CHUNKS = ROWS * D / 16;
#pragma unroll
  for (int c = tid; c < CHUNKS; c += NT) {
    uint32_t w0, w1, w2, w3;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(src8 + c * 16));
    const int r = (c * 16) / D, cc = ((c * 16) % D) / 8;
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst_plane + swz<D>(r, cc)), "r"(e4m3x2_to_bf16x2(w0)),
                 "r"(e4m3x2_to_bf16x2(w0 >> 16)), "r"(e4m3x2_to_bf16x2(w1)), "r"(e4m3x2_to_bf16x2(w1 >> 16)) : "memory");
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst_plane + swz<D>(r, cc + 1)), "r"(e4m3x2_to_bf16x2(w2)),
                 "r"(e4m3x2_to_bf16x2(w2 >> 16)), "r"(e4m3x2_to_bf16x2(w3)), "r"(e4m3x2_to_bf16x2(w3 >> 16)) : "memory");
  }
}

// S[16, NKEYS] (+)= Q[16, D] K[NKEYS, D]^T for one warp.  qf holds the A fragments of Q.
template <int D, int NKEYS>
LX_DEVICE void qk_tile(float (&sacc)[NKEYS / 8][4], const uint32_t (&qf)[D / 16][4], uint32_t k_smem, int lane) {
#pragma unroll
  for (int nt = 0; nt < NKEYS / 8; ++nt) {
#pragma unroll
    for (int q = 0; q < 4; ++q) sacc[nt][q] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ks += 2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(b0, b1, b2, b3, k_smem + swz<D>(nt * 8 + (lane & 7), 2 * ks + (lane >> 3)));
      mma_bf16_16816(sacc[nt], qf[ks], b0, b1);
      mma_bf16_16816(sacc[nt], qf[ks + 1], b2, b3);
    }
  }
}

// O[16, D] += P[16, NKEYS] V[NKEYS, D]
template <int D, int NKEYS>
LX_DEVICE void pv_tile(float (&oacc)[D / 8][4], const float (&sacc)[NKEYS / 8][4], uint32_t v_smem, int lane) {
#pragma unroll
  for (int kk = 0; kk < NKEYS / 16; ++kk) {
    uint32_t pa[4];
    pa[0] = pack_bf16x2(sacc[2 * kk][0], sacc[2 * kk][1]);
    pa[1] = pack_bf16x2(sacc[2 * kk][2], sacc[2 * kk][3]);
    pa[2] = pack_bf16x2(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
    pa[3] = pack_bf16x2(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
    for (int nd = 0; nd < D / 8; nd += 2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(b0, b1, b2, b3, v_smem + swz<D>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, nd + (lane >> 4)));
      mma_bf16_16816(oacc[nd], pa, b0, b1);
      mma_bf16_16816(oacc[nd + 1], pa, b2, b3);
    }
  }
}

// Online-softmax update for the two rows (lane/4 and lane/4 + 8) a thread owns.  `sacc` holds raw dot
// products on entry and probabilities on exit.  key0 = index of column 0; keys outside [lo, hi) are masked.
template <int D, int NKEYS>
LX_DEVICE void softmax_tile(float (&sacc)[NKEYS / 8][4], float (&oacc)[D / 8][4], float (&m)[2], float (&l)[2], int key0,
                            int lo0, int hi0, int lo1, int hi1, float scale, float softcap, int lane, float slope0 = 0.f,
                            float slope1 = 0.f) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NKEYS / 8; ++nt) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int key = key0 + nt * 8 + 2 * (lane & 3) + (q & 1);
      const int r = q >> 1;
      float s = sacc[nt][q] * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      // ALiBi: the bias -slope * (query position - key position) differs from slope * key position by a per-row constant,
      // which the softmax does not see
      s += (r == 0 ? slope0 : slope1) * (float)key;
      const bool ok = r == 0 ? (key >= lo0 && key < hi0) : (key >= lo1 && key < hi1);
      s = ok ? s : -INFINITY;
      sacc[nt][q] = s;
      mx[r] = fmaxf(mx[r], s);
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mnew[r] = fmaxf(m[r], mx[r]);
    corr[r] = (mnew[r] == -INFINITY) ? 1.f : exp2f((m[r] - mnew[r]) * kLog2e);
    m[r] = mnew[r];
    l[r] *= corr[r];
  }
#pragma unroll
  for (int nt = 0; nt < NKEYS / 8; ++nt) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = q >> 1;
      const float pz = (mnew[r] == -INFINITY) ? 0.f : exp2f((sacc[nt][q] - mnew[r]) * kLog2e);
      sacc[nt][q] = pz;
      l[r] += pz;
    }
  }
#pragma unroll
  for (int nd = 0; nd < D / 8; ++nd) {
    oacc[nd][0] *= corr[0]; oacc[nd][1] *= corr[0];
    oacc[nd][2] *= corr[1]; oacc[nd][3] *= corr[1];
  }
}

// ------------------------------------------------------------------------------------------------
// Decode
// ------------------------------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* q;     // [T, ldq], head h at column h * D
  long long ldq;
  const __nv_bfloat16* kv;    // cache of this layer
  const int* block_tables;    // [T, max_blocks]
  int max_blocks;
  const int* ctx_lens;        // [T] number of keys visible to the token (includes itself); <= 0: skip row
  __nv_bfloat16* out;         // [T, ldo]
  long long ldo;
  float* part_o;              // split-KV partials [T, nh, nsplit, D]
  float* part_lse;            // [T, nh, nsplit]
  int nh, nkv, group, gchunks;
  int window;                 // <= 0: none
  float scale, softcap;
  int nsplit;
  const float* alibi;         // [nh] ALiBi slopes, or null
  float v_scale;              // fp8 cache: multiplies the output (the K scale is folded into `scale` by the host)
};

// NW warps per CTA split the pages of a (row, KV head): four for long contexts; two, so that two CTAs fit an SM and one streams
// while the other starts or combines, for the short contexts of a large decode batch.
template <int D, int STAGES, bool KV8, int NW>
__global__ void __launch_bounds__(32 * NW) attn_decode_kernel(const DecodeParams p) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  extern __shared__ __align__(1024) uint8_t dsm[];
  constexpr int PLANE = kPage * D * 2;
  constexpr int PLANE8 = kPage * D;
  constexpr int STAGE = KV8 ? 2 * PLANE8 : 2 * PLANE;
  constexpr int WARP_BYTES = STAGES * STAGE + (KV8 ? 2 * PLANE : 0);     // fp8: staged bytes + one expanded K and V plane
  const int t = blockIdx.x;
  const int kvh = blockIdx.y / p.gchunks, gc = blockIdx.y % p.gchunks;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = p.ctx_lens[t];
  const int g0 = gc * 16;
  const int grows = min(16, p.group - g0);
  const int head0 = kvh * p.group + g0;

  int key_lo = 0;
  if (p.window > 0 && ctx > p.window) key_lo = ctx - p.window;
  const int page_lo = key_lo / kPage;
  const int page_hi = ctx > 0 ? (ctx + kPage - 1) / kPage : 0;
  const int npages = max(page_hi - page_lo, 0);
  const int per_split = (npages + p.nsplit - 1) / p.nsplit;
  const int pb = page_lo + split * per_split;
  const int pe = min(pb + per_split, page_hi);

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }

  // Q fragments straight from global memory (row = head in group, zero beyond the group).
  uint32_t qf[D / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    const __nv_bfloat16* q0 = p.q + (long long)t * p.ldq + (long long)(head0 + r0) * D;
    const __nv_bfloat16* q1 = p.q + (long long)t * p.ldq + (long long)(head0 + r1) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int c = ks * 16 + 2 * (lane & 3);
      qf[ks][0] = r0 < grows ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
      qf[ks][1] = r1 < grows ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
      qf[ks][2] = r0 < grows ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
      qf[ks][3] = r1 < grows ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
    }
  }

  const uint32_t wbase = smem_u32(dsm) + warp * WARP_BYTES;
  const uint32_t wwork = wbase + STAGES * STAGE;
  const int* bt = p.block_tables + (long long)t * p.max_blocks;
  float slope0 = 0.f, slope1 = 0.f;
  if (p.alibi != nullptr) {
    const int r0 = lane >> 2, r1 = r0 + 8;
    slope0 = r0 < grows ? p.alibi[head0 + r0] : 0.f;
    slope1 = r1 < grows ? p.alibi[head0 + r1] : 0.f;
  }
  const int my_first = pb + warp;
  const int my_count = my_first < pe ? (pe - my_first + NW - 1) / NW : 0;

  auto issue = [&](int i) {
    if (i < my_count) {
      const int page = my_first + NW * i;
      const long long blk = bt[page];
      const uint32_t sb = wbase + (i % STAGES) * STAGE;
      if constexpr (KV8) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.kv) + ((blk * p.nkv + kvh) * 2) * (long long)(kPage * D);
        load_plane8<D, 2 * kPage, 32>(sb, src, lane, true);            // the K plane and the V plane are one contiguous run
      } else {
        const __nv_bfloat16* src = p.kv + ((blk * p.nkv + kvh) * 2) * (long long)(kPage * D);
        load_plane<D, kPage, 32>(sb, src, lane, true);
        load_plane<D, kPage, 32>(sb + PLANE, src + kPage * D, lane, true);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue(s);

  for (int i = 0; i < my_count; ++i) {
    issue(i + STAGES - 1);
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    uint32_t sb = wbase + (i % STAGES) * STAGE;
    if constexpr (KV8) {
      expand_plane8<D, kPage, 32>(wwork, sb, lane);
      expand_plane8<D, kPage, 32>(wwork + PLANE, sb + PLANE8, lane);
      __syncwarp();
      sb = wwork;
    }
    const int page = my_first + NW * i;
    float sacc[kPage / 8][4];
    qk_tile<D, kPage>(sacc, qf, sb, lane);
    softmax_tile<D, kPage>(sacc, oacc, m, l, page * kPage, key_lo, ctx, key_lo, ctx, p.scale, p.softcap, lane, slope0, slope1);
    pv_tile<D, kPage>(oacc, sacc, sb + PLANE, lane);
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- combine the four warps through shared memory (pipeline buffers are free now)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  float* so = reinterpret_cast<float*>(dsm);            // [NW][16][D]
  float* sm = so + NW * 16 * D;                          // [NW][16]
  float* sl = sm + NW * 16;                              // [NW][16]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int nd = 0; nd < D / 8; ++nd) {
      const int c = nd * 8 + 2 * (lane & 3);
      *reinterpret_cast<float2*>(so + (warp * 16 + r0) * D + c) = make_float2(oacc[nd][0], oacc[nd][1]);
      *reinterpret_cast<float2*>(so + (warp * 16 + r1) * D + c) = make_float2(oacc[nd][2], oacc[nd][3]);
    }
    if ((lane & 3) == 0) {
      sm[warp * 16 + r0] = m[0]; sm[warp * 16 + r1] = m[1];
      sl[warp * 16 + r0] = l[0]; sl[warp * 16 + r1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < grows * D; idx += 32 * NW) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, sm[w * 16 + g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = sm[w * 16 + g];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f((mw - M) * kLog2e);
      num += wgt * so[(w * 16 + g) * D + d];
      den += wgt * sl[w * 16 + g];
    }
    const float o = (den > 0.f ? num / den : 0.f) * (KV8 ? p.v_scale : 1.f);
    const int head = head0 + g;
    if (p.nsplit == 1) {
      p.out[(long long)t * p.ldo + (long long)head * D + d] = __float2bfloat16(o);
    } else {
      const long long pi = ((long long)t * p.nh + head) * p.nsplit + split;
      p.part_o[pi * D + d] = o;
      if (d == 0) p.part_lse[pi] = den > 0.f ? M + __logf(den) : -INFINITY;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(D) attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                                         __nv_bfloat16* __restrict__ out, long long ldo, int nh, int nsplit) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const long long base = ((long long)t * nh + h) * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_lse[base + s]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ls = part_lse[base + s];
    const float w = (ls == -INFINITY) ? 0.f : __expf(ls - M);
    num += w * part_o[(base + s) * D + d];
    den += w;
  }
  out[(long long)t * ldo + (long long)h * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

// ------------------------------------------------------------------------------------------------
// Prefill: 64 queries x 1 head per CTA (16 query rows per warp), 64-key tiles = two cache pages.
// ------------------------------------------------------------------------------------------------
struct PrefillParams {
  const __nv_bfloat16* q;     // [T, ldq]
  long long ldq;
  const __nv_bfloat16* kv;
  const int* block_tables;    // [B, max_blocks]
  int max_blocks;
  const int* cu_q;            // [B + 1] start of each sequence's chunk in the ragged token dimension
  const int* cache_lens;      // [B] keys already cached before this chunk
  const int* tile_seq;        // [num_tiles] sequence of each 64-query tile
  const int* tile_q0;         // [num_tiles] first query (within the chunk) of the tile
  __nv_bfloat16* out;
  long long ldo;
  int nh, nkv;
  int window;
  float scale, softcap;
  const float* alibi;         // [nh] ALiBi slopes, or null
  float v_scale;              // fp8 cache: multiplies the output
};

template <int D, bool KV8>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const PrefillParams p) {
  pdl_trigger();
  pdl_wait();      // every block waits, also those that return early below
  extern __shared__ __align__(1024) uint8_t psm[];
  constexpr int KT = 64;                         // keys per tile
  constexpr int PLANE = kPage * D * 2;           // one page of K or V
  constexpr int PLANE8 = kPage * D;
  constexpr int STAGE = KV8 ? 4 * PLANE8 : 4 * PLANE;        // K page0, K page1, V page0, V page1 (fp8: K0 V0 K1 V1 as bytes)
  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (p.nh / p.nkv);
  const int b = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int qlen = p.cu_q[b + 1] - p.cu_q[b];
  const int cache = p.cache_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = p.block_tables + (long long)b * p.max_blocks;

  // rows owned by this thread
  const int qr0 = q0 + warp * 16 + (lane >> 2), qr1 = qr0 + 8;
  const long long tok0 = (long long)p.cu_q[b] + qr0, tok1 = (long long)p.cu_q[b] + qr1;
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int c = ks * 16 + 2 * (lane & 3);
    const __nv_bfloat16* a0 = p.q + tok0 * p.ldq + (long long)head * D + c;
    const __nv_bfloat16* a1 = p.q + tok1 * p.ldq + (long long)head * D + c;
    qf[ks][0] = qr0 < qlen ? *reinterpret_cast<const uint32_t*>(a0) : 0u;
    qf[ks][1] = qr1 < qlen ? *reinterpret_cast<const uint32_t*>(a1) : 0u;
    qf[ks][2] = qr0 < qlen ? *reinterpret_cast<const uint32_t*>(a0 + 8) : 0u;
    qf[ks][3] = qr1 < qlen ? *reinterpret_cast<const uint32_t*>(a1 + 8) : 0u;
  }
  // visible key range per row: [lo, hi) with hi = position + 1
  const int pos0 = cache + qr0, pos1 = cache + qr1;
  const int hi0 = qr0 < qlen ? pos0 + 1 : 0, hi1 = qr1 < qlen ? pos1 + 1 : 0;
  const int lo0 = (p.window > 0 && hi0 > p.window) ? hi0 - p.window : 0;
  const int lo1 = (p.window > 0 && hi1 > p.window) ? hi1 - p.window : 0;

  // key tiles needed by the CTA
  const int last_q = min(q0 + 63, qlen - 1);
  const int key_hi = cache + last_q + 1;
  int key_lo = 0;
  if (p.window > 0) key_lo = max(cache + q0 + 1 - p.window, 0);
  const int t_lo = key_lo / KT, t_hi = (key_hi + KT - 1) / KT;
  const int total_pages = (key_hi + kPage - 1) / kPage;

  const uint32_t base = smem_u32(psm);
  auto issue = [&](int kt) {
    if (kt < t_hi) {
      const uint32_t sb = base + (kt & 1) * STAGE;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int page = kt * 2 + h;
        const bool valid = page < total_pages;
        const long long blk = valid ? bt[page] : 0;
        if constexpr (KV8) {
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.kv) + ((blk * p.nkv + kvh) * 2) * (long long)(kPage * D);
          load_plane8<D, 2 * kPage, 128>(sb + h * 2 * PLANE8, src, threadIdx.x, valid);
        } else {
          const __nv_bfloat16* src = p.kv + ((blk * p.nkv + kvh) * 2) * (long long)(kPage * D);
          load_plane<D, kPage, 128>(sb + h * PLANE, src, threadIdx.x, valid);
          load_plane<D, kPage, 128>(sb + (2 + h) * PLANE, src + kPage * D, threadIdx.x, valid);
        }
      }
    }
    cp_async_commit();
  };
  const uint32_t work = base + 2 * STAGE;        // fp8: the expanded bf16 planes of the tile being multiplied

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float oacc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
  const float slope = p.alibi != nullptr ? p.alibi[head] : 0.f;

  issue(t_lo);
  for (int kt = t_lo; kt < t_hi; ++kt) {
    issue(kt + 1);
    cp_async_wait<1>();
    __syncthreads();
    uint32_t sb = base + (kt & 1) * STAGE;
    if constexpr (KV8) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        expand_plane8<D, kPage, 128>(work + h * PLANE, sb + h * 2 * PLANE8, threadIdx.x);
        expand_plane8<D, kPage, 128>(work + (2 + h) * PLANE, sb + h * 2 * PLANE8 + PLANE8, threadIdx.x);
      }
      __syncthreads();
      sb = work;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float sacc[kPage / 8][4];
      qk_tile<D, kPage>(sacc, qf, sb + h * PLANE, lane);
      softmax_tile<D, kPage>(sacc, oacc, m, l, kt * KT + h * kPage, lo0, hi0, lo1, hi1, p.scale, p.softcap, lane, slope, slope);
      pv_tile<D, kPage>(oacc, sacc, sb + (2 + h) * PLANE, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  const float vs = KV8 ? p.v_scale : 1.f;
  const float inv0 = l[0] > 0.f ? vs / l[0] : 0.f, inv1 = l[1] > 0.f ? vs / l[1] : 0.f;
#pragma unroll
  for (int nd = 0; nd < D / 8; ++nd) {
    const int c = nd * 8 + 2 * (lane & 3);
    if (qr0 < qlen)
      *reinterpret_cast<uint32_t*>(p.out + tok0 * p.ldo + (long long)head * D + c) = pack_bf16x2(oacc[nd][0] * inv0, oacc[nd][1] * inv0);
    if (qr1 < qlen)
      *reinterpret_cast<uint32_t*>(p.out + tok1 * p.ldo + (long long)head * D + c) = pack_bf16x2(oacc[nd][2] * inv1, oacc[nd][3] * inv1);
  }
}

template <int D, int STAGES, bool KV8, int NW>
static int launch_decode_nw(const DecodeParams& p, int T, cudaStream_t s) {
  constexpr int SMEM = KV8 ? NW * (STAGES * 2 * kPage * D + 2 * kPage * D * 2) : NW * STAGES * 2 * kPage * D * 2;
  static_assert(SMEM >= (NW * 16 * D + 2 * NW * 16) * 4, "combine buffer must fit in the pipeline buffers");
  static bool configured[64] = {false};          // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, STAGES, KV8, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(T, p.nkv * p.gchunks, p.nsplit);
  launch_pdl(attn_decode_kernel<D, STAGES, KV8, NW>, grid, dim3(32 * NW), (size_t)SMEM, s, p);
  if (p.nsplit > 1) {
    dim3 g2(T, p.nh);
    launch_pdl(attn_combine_kernel<D>, g2, dim3(D), 0, s, p.part_o, p.part_lse, p.out, p.ldo, p.nh, p.nsplit);
  }
  return -(int)cudaGetLastError();
}

template <int D, int STAGES, bool KV8>
static int launch_decode(const DecodeParams& p, int T, cudaStream_t s) {
  // Enough CTAs for several waves over the GPU: two warps per CTA, two CTAs per SM (their start-up and combine phases overlap the
  // other's streaming).  Few CTAs (small batches, split contexts): four warps each, so that one CTA keeps more pages in flight.
  static int force = -1;
  if (force < 0) {
    const char* e = getenv("LORAX_ATTN_DECODE_WARPS");
    force = e ? atoi(e) : 0;
  }
  const long long ctas = (long long)T * p.nkv * p.gchunks * p.nsplit;
  const bool two = force == 2 || (force != 4 && ctas >= 2 * 148);
  if (two) return launch_decode_nw<D, STAGES, KV8, 2>(p, T, s);
  return launch_decode_nw<D, STAGES, KV8, 4>(p, T, s);
}

template <int D, bool KV8>
static int launch_prefill(const PrefillParams& p, int num_tiles, cudaStream_t s) {
  constexpr int SMEM = KV8 ? 2 * 4 * kPage * D + 4 * kPage * D * 2 : 2 * 4 * kPage * D * 2;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D, KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid(num_tiles, p.nh);
  launch_pdl(attn_prefill_kernel<D, KV8>, grid, dim3(128), (size_t)SMEM, s, p);
  return -(int)cudaGetLastError();
}

}  // namespace lx

extern "C" {

int lx_attn_page_size() { return lx::kPage; }

// part_o / part_lse are only touched when nsplit > 1: sizes T*nh*nsplit*D and T*nh*nsplit floats.
int lx_attn_decode_alibi(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                         void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                         float softcap, int nsplit, const float* alibi, void* stream);
int lx_attn_prefill_alibi(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                          const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                          int nkv, int d, int window, float scale, float softcap, const float* alibi, void* stream);

int lx_attn_decode(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                   void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                   float softcap, int nsplit, void* stream) {
  return lx_attn_decode_alibi(q, ldq, kv, block_tables, max_blocks, ctx_lens, out, ldo, part_o, part_lse, T, nh, nkv, d, window, scale,
                              softcap, nsplit, nullptr, stream);
}

static int attn_decode_impl(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                            void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                            float softcap, int nsplit, const float* alibi, bool kv8, float k_scale, float v_scale, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (nh % nkv != 0) return -1;
  DecodeParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.ldq = ldq;
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.ctx_lens = ctx_lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.part_o = part_o; p.part_lse = part_lse;
  p.nh = nh; p.nkv = nkv; p.group = nh / nkv; p.gchunks = (p.group + 15) / 16;
  p.window = window; p.scale = kv8 ? scale * k_scale : scale; p.softcap = softcap; p.alibi = alibi;
  p.v_scale = v_scale;
  p.nsplit = nsplit < 1 ? 1 : nsplit;
  if (p.nsplit > 1 && (part_o == nullptr || part_lse == nullptr)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (kv8) {
    if (d == 128) return launch_decode<128, 3, true>(p, T, s);
    if (d == 64) return launch_decode<64, 4, true>(p, T, s);
    return -3;
  }
  if (d == 128) return launch_decode<128, 3, false>(p, T, s);
  if (d == 64) return launch_decode<64, 4, false>(p, T, s);
  return -3;
}

// `alibi`: [nh] fp32 slopes on the device (BLOOM, MPT), or null.
int lx_attn_decode_alibi(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                         void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                         float softcap, int nsplit, const float* alibi, void* stream) {
  return attn_decode_impl(q, ldq, kv, block_tables, max_blocks, ctx_lens, out, ldo, part_o, part_lse, T, nh, nkv, d, window, scale, softcap,
                          nsplit, alibi, false, 1.f, 1.f, stream);
}

// The same over an e4m3 cache: stored value * k_scale (v_scale) is the key (value).
int lx_attn_decode_kv8(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                       void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                       float softcap, int nsplit, const float* alibi, float k_scale, float v_scale, void* stream) {
  return attn_decode_impl(q, ldq, kv, block_tables, max_blocks, ctx_lens, out, ldo, part_o, part_lse, T, nh, nkv, d, window, scale, softcap,
                          nsplit, alibi, true, k_scale, v_scale, stream);
}

int lx_attn_prefill(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                    const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                    int nkv, int d, int window, float scale, float softcap, void* stream) {
  return lx_attn_prefill_alibi(q, ldq, kv, block_tables, max_blocks, cu_q, cache_lens, tile_seq, tile_q0, num_tiles, out, ldo, nh, nkv, d,
                               window, scale, softcap, nullptr, stream);
}

static int attn_prefill_impl(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                             const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                             int nkv, int d, int window, float scale, float softcap, const float* alibi, bool kv8, float k_scale,
                             float v_scale, void* stream) {
  using namespace lx;
  if (num_tiles <= 0) return 0;
  if (nh % nkv != 0) return -1;
  PrefillParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q); p.ldq = ldq;
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.cu_q = cu_q; p.cache_lens = cache_lens;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.nh = nh; p.nkv = nkv; p.window = window; p.scale = kv8 ? scale * k_scale : scale; p.softcap = softcap; p.alibi = alibi;
  p.v_scale = v_scale;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (kv8) {
    if (d == 128) return launch_prefill<128, true>(p, num_tiles, s);
    if (d == 64) return launch_prefill<64, true>(p, num_tiles, s);
    return -3;
  }
  if (d == 128) return launch_prefill<128, false>(p, num_tiles, s);
  if (d == 64) return launch_prefill<64, false>(p, num_tiles, s);
  return -3;
}

int lx_attn_prefill_alibi(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                          const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                          int nkv, int d, int window, float scale, float softcap, const float* alibi, void* stream) {
  return attn_prefill_impl(q, ldq, kv, block_tables, max_blocks, cu_q, cache_lens, tile_seq, tile_q0, num_tiles, out, ldo, nh, nkv, d, window,
                           scale, softcap, alibi, false, 1.f, 1.f, stream);
}

int lx_attn_prefill_kv8(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                        const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                        int nkv, int d, int window, float scale, float softcap, const float* alibi, float k_scale, float v_scale,
                        void* stream) {
  return attn_prefill_impl(q, ldq, kv, block_tables, max_blocks, cu_q, cache_lens, tile_seq, tile_q0, num_tiles, out, ldo, nh, nkv, d, window,
                           scale, softcap, alibi, true, k_scale, v_scale, stream);
}

}  // extern "C"
