// Ragged causal prefill attention over the paged KV cache on the 5th-generation tensor cores.
//
// One CTA = one 64-query tile of one sequence x TWO query heads of the same KV group: the 128 rows of a tcgen05 M tile are
// (head, query) pairs, so a K / V block is staged once for both heads.  Keys are walked in blocks of 128 (four cache pages):
//
//   loader  (warp 0, one lane)  Q by TMA from the projection output; K and V pages by TMA straight from the paged cache
//                               through one 5-D tensor map {d, slot, K|V, kv head, block}: the block table supplies the last
//                               coordinate, so pages need not be contiguous; a two-stage ring
//   MMA     (warp 1, one lane)  S = Q K^T into TMEM (double buffered), then O_j = P_j V_j into TMEM (double buffered); P comes
//                               back from the softmax warps through shared memory as a K-major operand, V is used as stored
//                               (token-major = the "MN-major" form of the B operand); S of block j+1 is issued before P_j V_j,
//                               so the tensor core works on the next scores while the softmax of this block runs
//   softmax (warps 2..5)        one thread per row: scores from TMEM with tcgen05.ld, scale / softcap / ALiBi / causal and
//                               window mask, running max and sum, exp2, P as bf16 into the swizzled operand tile; the
//                               per-block products O_j come back from TMEM and are folded into fp32 registers with the
//                               usual rescaling, so nothing in TMEM ever has to be rescaled
//
// Plain, chunked and prefix-cached prefill are one path: `cache_lens` says how many keys precede the chunk.  It replaces the
// flash-attn-2 varlen call of the reference (server/lorax_server/utils/flash_attn.py:180-201) and the mma.sync kernel in
// attention.cu, which stays for head sizes and group sizes this one does not take (d != 128, odd heads per KV head).
// Every wait is bounded and reports through the status word.
#include "common.cuh"

namespace lx {

constexpr int kFaPage = 32;
constexpr int kFaQ = 64;            // queries per CTA (per head)
constexpr int kFaKeys = 128;        // keys per block
constexpr int kFaD = 128;
constexpr int kFaThreads = 192;
constexpr float kFaLog2e = 1.4426950408889634f;

struct FaParams {
  const int* block_tables;
  int max_blocks;
  const int* cu_q;
  const int* cache_lens;
  const int* tile_seq;
  const int* tile_q0;
  __nv_bfloat16* out;
  long long ldo;
  int nh, nkv, group;
  int window;
  float scale, softcap;
  const float* alibi;
  int* status;
};

struct FaSmem {
  static constexpr int kQBytes = 128 * kFaD * 2;             // two 64-wide halves of [128 rows x 64]
  static constexpr int kKBytes = kFaKeys * kFaD * 2;
  static constexpr int kVBytes = kFaKeys * kFaD * 2;
  static constexpr int kPBytes = 128 * kFaKeys * 2;
  static constexpr int kStage = kKBytes + kVBytes;
  static constexpr int kTotal = kQBytes + 2 * kStage + kPBytes + 512 + 1024;
};

// 5-D tiled load: the paged cache {d, slot in page, K|V, kv head, block}.
LX_DEVICE void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
LX_DEVICE void mbar_arrive_cnt(uint64_t* bar) { mbar_arrive(bar); }

LX_DEVICE float fa_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One score: scale, optional tanh cap, optional ALiBi bias, in the log2 domain (the softmax uses exp2).
LX_DEVICE float fa_score(float s, float scale_l2, float softcap, float scale, float slope_l2, int key) {
  float t;
  if (softcap > 0.f) t = softcap * tanhf(s * scale / softcap) * kFaLog2e;
  else t = s * scale_l2;
  return fmaf(slope_l2, (float)key, t);
}

// Maximum over the 128 scores of a row (log2 domain).  PLAIN: no cap, no bias, so max(s) * scale is the maximum; MASK: keys
// outside [lo, hi) do not count.
template <bool PLAIN, bool MASK>
LX_DEVICE float fa_block_max(uint32_t ts, int kb0, int lo, int hi, float scale_l2, float softcap, float scale, float slope_l2) {
  float bm = -INFINITY;
#pragma unroll 1
  for (int c = 0; c < kFaKeys; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(ts + (uint32_t)c, r);
    tc_wait_ld();
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      float t = PLAIN ? __uint_as_float(r[q]) : fa_score(__uint_as_float(r[q]), scale_l2, softcap, scale, slope_l2, kb0 + c + q);
      if (MASK) {
        const int key = kb0 + c + q;
        t = (key >= lo && key < hi) ? t : -INFINITY;
      }
      bm = fmaxf(bm, t);
    }
  }
  return PLAIN ? bm * scale_l2 : bm;
}

// p = exp2(score - m_new) for the 128 keys of the block -> bf16, written as this row of the K-major, 128-byte-swizzled operand
// tile; returns the row sum.
template <bool PLAIN, bool MASK>
LX_DEVICE float fa_block_probs(uint32_t ts, uint8_t* prow, int row, int kb0, int lo, int hi, float m_new, float scale_l2, float softcap,
                               float scale, float slope_l2) {
  float sum = 0.f;
  const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
  const bool dead = (m_new == -INFINITY);
#pragma unroll 1
  for (int c = 0; c < kFaKeys; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(ts + (uint32_t)c, r);
    tc_wait_ld();
    uint32_t pk[16];
#pragma unroll
    for (int q = 0; q < 32; q += 2) {
      float pv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float sraw = __uint_as_float(r[q + u]);
        float e = PLAIN ? fa_ex2(fmaf(sraw, scale_l2, neg_m)) : fa_ex2(fa_score(sraw, scale_l2, softcap, scale, slope_l2, kb0 + c + q + u) + neg_m);
        if (MASK) {
          const int key = kb0 + c + q + u;
          e = (key >= lo && key < hi && !dead) ? e : 0.f;
        }
        pv[u] = e;
      }
      sum += pv[0] + pv[1];
      pk[q >> 1] = pack_bf16x2(pv[0], pv[1]);
    }
    uint8_t* half = prow + (c >> 6) * 16384;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const int chunk = ((c & 63) >> 3) + ch;
      *reinterpret_cast<uint4*>(half + ((chunk ^ (row & 7)) << 4)) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
    }
  }
  return sum;
}

__global__ void __launch_bounds__(kFaThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv, const FaParams p) {
  pdl_trigger();
  using S = FaSmem;
  extern __shared__ uint8_t fa_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  uint8_t* skv = smem + S::kQBytes;
  uint8_t* sp = skv + 2 * S::kStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp + S::kPBytes);
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // 2
  uint64_t* kv_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;        // 2
  uint64_t* s_empty = bars + 7;       // 2  (128 arrivals)
  uint64_t* p_full = bars + 9;        // 1  (128 arrivals)
  uint64_t* p_empty = bars + 10;      // 1
  uint64_t* pv_full = bars + 11;      // 2
  uint64_t* pv_empty = bars + 13;     // 2  (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;      // later tiles of a sequence see more keys: start the long ones first
  const int h0 = blockIdx.y * 2;                 // first of the two query heads
  const int kvh = h0 / p.group;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 128);
      mbar_init(&pv_full[i], 1); mbar_init(&pv_empty[i], 128);
    }
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_kv);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  const int b = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int tok_base = p.cu_q[b];
  const int qlen = p.cu_q[b + 1] - tok_base;
  const int cache = p.cache_lens[b];
  // keys the tile needs: [key_lo, key_hi)
  const int last_q = min(q0 + kFaQ - 1, qlen - 1);
  const int key_hi = cache + last_q + 1;
  const int key_lo = p.window > 0 ? max(cache + q0 + 1 - p.window, 0) : 0;
  const int t_lo = key_lo / kFaKeys;
  const int nblk = max((key_hi + kFaKeys - 1) / kFaKeys - t_lo, 0);
  const int total_pages = (key_hi + kFaPage - 1) / kFaPage;

  if (warp == 0) {
    if (lane == 0 && nblk > 0) {
      // Q: rows 0..63 = head h0, rows 64..127 = head h0 + 1; two 64-wide halves of d
      mbar_expect_tx(q_full, (uint32_t)S::kQBytes);
      for (int g = 0; g < 2; ++g)
        for (int hf = 0; hf < 2; ++hf)
          tma_load_2d(sq + hf * 16384 + g * 8192, &tmap_q, q_full, (h0 + g) * kFaD + hf * 64, tok_base + q0);
      const int* bt = p.block_tables + (long long)b * p.max_blocks;
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag)) { report_status(p.status, kTimeoutEmptyBarrier, tile); *abort_flag = 1; break; }
        uint8_t* sk = skv + st * S::kStage;
        uint8_t* sv = sk + S::kKBytes;
        mbar_expect_tx(&kv_full[st], (uint32_t)S::kStage);
        for (int pg = 0; pg < 4; ++pg) {
          const int page = (t_lo + j) * 4 + pg;
          const int blk = (page < total_pages && page < p.max_blocks) ? bt[page] : 0;      // a page past the keys reads block 0: masked, but finite
          for (int hf = 0; hf < 2; ++hf) {
            tma_load_5d(sk + hf * 16384 + pg * 4096, &tmap_kv, &kv_full[st], hf * 64, 0, 0, kvh, blk);
            tma_load_5d(sv + hf * 16384 + pg * 4096, &tmap_kv, &kv_full[st], hf * 64, 0, 1, kvh, blk);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && nblk > 0) {
      const uint32_t idesc_s = make_idesc(128, kFaKeys, kFmtBF16, kFmtBF16);
      const uint32_t idesc_pv = make_idesc(128, kFaD, kFmtBF16, kFmtBF16, 0, 1);          // B (= V) is MN-major
      const uint32_t sq_a = smem_u32(sq), sp_a = smem_u32(sp);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (!ok) { report_status(p.status, kTimeoutFullBarrier, tile); *abort_flag = 1; }
      auto do_pv = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(p_full, i & 1, abort_flag) || !mbar_wait(&pv_empty[st], ((i >> 1) & 1) ^ 1, abort_flag)) {
          report_status(p.status, kTimeoutTmemEmpty, tile); *abort_flag = 1; return false;
        }
        tc_fence_after();
        const uint32_t sv_a = smem_u32(skv + st * S::kStage + S::kKBytes);
        const uint32_t tmem_o = tmem_base + 256u + (uint32_t)(st * 128);
#pragma unroll
        for (int ks = 0; ks < kFaKeys / 16; ++ks) {
          const uint64_t da = make_desc_k_sw128(sp_a + (uint32_t)((ks >> 2) * 16384)) + (uint64_t)((ks & 3) * 2);
          const uint64_t db = make_desc_mn_sw128(sv_a + (uint32_t)(ks * 2048), 16384, 1024);
          umma_f16_ss(tmem_o, da, db, idesc_pv, ks > 0 ? 1u : 0u);
        }
        tc_commit(&pv_full[st]);
        tc_commit(p_empty);
        tc_commit(&kv_empty[st]);
        return true;
      };
      for (int j = 0; ok && j < nblk; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_full[st], (j >> 1) & 1, abort_flag) || !mbar_wait(&s_empty[st], ((j >> 1) & 1) ^ 1, abort_flag)) {
          report_status(p.status, kTimeoutFullBarrier, tile); *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t sk_a = smem_u32(skv + st * S::kStage);
        const uint32_t tmem_s = tmem_base + (uint32_t)(st * 128);
#pragma unroll
        for (int ks = 0; ks < kFaD / 16; ++ks) {
          const uint64_t da = make_desc_k_sw128(sq_a + (uint32_t)((ks >> 2) * 16384)) + (uint64_t)((ks & 3) * 2);
          const uint64_t db = make_desc_k_sw128(sk_a + (uint32_t)((ks >> 2) * 16384)) + (uint64_t)((ks & 3) * 2);
          umma_f16_ss(tmem_s, da, db, idesc_s, ks > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[st]);
        if (j > 0) ok = do_pv(j - 1);
      }
      if (ok) do_pv(nblk - 1);
    }
    __syncwarp();
  } else if (nblk > 0) {
    // ------------------------------------------------------------------ softmax warps: one row per thread
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int head = h0 + (row >> 6);
    const int qi = q0 + (row & 63);
    const bool row_ok = qi < qlen;
    const int hi = row_ok ? cache + qi + 1 : 0;
    const int lo = (p.window > 0 && hi > p.window) ? hi - p.window : 0;
    // block-level bounds: a block whose keys every row of the tile sees needs no mask
    const int hi_min = cache + q0 + 1;
    const int lo_max = (p.window > 0 && key_hi > p.window) ? key_hi - p.window : 0;
    const bool rows_all_valid = (q0 + kFaQ <= qlen);
    const float scale_l2 = p.scale * kFaLog2e;
    const float slope_l2 = p.alibi != nullptr ? p.alibi[head] * kFaLog2e : 0.f;
    const bool plain = p.softcap <= 0.f && p.alibi == nullptr;       // scores are s * scale: the maximum can be taken before scaling
    const uint32_t trow = tmem_base + ((uint32_t)(quad * 32) << 16);
    uint8_t* prow = sp + row * 128;

    float m = -INFINITY, l = 0.f;
    float o[kFaD];
#pragma unroll
    for (int i = 0; i < kFaD; ++i) o[i] = 0.f;
    bool alive = true;

    for (int j = 0; j < nblk && alive; ++j) {
      const int st = j & 1;
      const int kb0 = (t_lo + j) * kFaKeys;
      if (!mbar_wait(&s_full[st], (j >> 1) & 1, abort_flag)) { report_status(p.status, kTimeoutTmemFull, tile); *abort_flag = 1; alive = false; break; }
      tc_fence_after();
      const bool need_mask = !(rows_all_valid && kb0 + kFaKeys <= hi_min && kb0 >= lo_max);
      const uint32_t ts = trow + (uint32_t)(st * 128);
      // pass 1: block maximum of this row (log2 domain)
      float bm;
      if (plain) bm = need_mask ? fa_block_max<true, true>(ts, kb0, lo, hi, scale_l2, p.softcap, p.scale, slope_l2)
                                : fa_block_max<true, false>(ts, kb0, lo, hi, scale_l2, p.softcap, p.scale, slope_l2);
      else bm = fa_block_max<false, true>(ts, kb0, lo, hi, scale_l2, p.softcap, p.scale, slope_l2);
      const float m_new = fmaxf(m, bm);
      const float alpha = (m_new == -INFINITY) ? 1.f : fa_ex2(m - m_new);
      // the P tile is free once the MMAs of the previous block have read it
      if (!mbar_wait(p_empty, (j & 1) ^ 1, abort_flag)) { report_status(p.status, kTimeoutTmemEmpty, tile); *abort_flag = 1; alive = false; break; }
      // pass 2: probabilities -> bf16 operand tile, row sum
      float sum;
      if (plain) sum = need_mask ? fa_block_probs<true, true>(ts, prow, row, kb0, lo, hi, m_new, scale_l2, p.softcap, p.scale, slope_l2)
                                 : fa_block_probs<true, false>(ts, prow, row, kb0, lo, hi, m_new, scale_l2, p.softcap, p.scale, slope_l2);
      else sum = fa_block_probs<false, true>(ts, prow, row, kb0, lo, hi, m_new, scale_l2, p.softcap, p.scale, slope_l2);
      tc_fence_before();
      mbar_arrive(&s_empty[st]);
      fence_proxy_async_smem();
      mbar_arrive(p_full);
      l = l * alpha + sum;
      // fold the previous block's product in: o = (o + O_{j-1}) * alpha
      if (j > 0) {
        const int ps = (j - 1) & 1;
        if (!mbar_wait(&pv_full[ps], ((j - 1) >> 1) & 1, abort_flag)) { report_status(p.status, kTimeoutTmemFull, tile); *abort_flag = 1; alive = false; break; }
        tc_fence_after();
        const bool same_max = __all_sync(0xffffffffu, alpha == 1.f);      // no row of the warp saw a new maximum: nothing to rescale
#pragma unroll
        for (int c = 0; c < kFaD; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(trow + (uint32_t)(256 + ps * 128 + c), r);
          tc_wait_ld();
          if (same_max) {
#pragma unroll
            for (int q = 0; q < 32; ++q) o[c + q] += __uint_as_float(r[q]);
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) o[c + q] = (o[c + q] + __uint_as_float(r[q])) * alpha;
          }
        }
        tc_fence_before();
        mbar_arrive(&pv_empty[ps]);
      }
      m = m_new;
    }
    if (alive) {
      const int ps = (nblk - 1) & 1;
      if (mbar_wait(&pv_full[ps], ((nblk - 1) >> 1) & 1, abort_flag)) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* orow = p.out + (long long)(tok_base + qi) * p.ldo + (long long)head * kFaD;
#pragma unroll
        for (int c = 0; c < kFaD; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(trow + (uint32_t)(256 + ps * 128 + c), r);
          tc_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 32; q += 8) {
              uint32_t w[4];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                w[u] = pack_bf16x2((o[c + q + 2 * u] + __uint_as_float(r[q + 2 * u])) * inv, (o[c + q + 2 * u + 1] + __uint_as_float(r[q + 2 * u + 1])) * inv);
              *reinterpret_cast<uint4*>(orow + c + q) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      } else {
        report_status(p.status, kTimeoutTmemFull, tile);
        *abort_flag = 1;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static FaEncodeFn fa_encode_fn() {
  static FaEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<FaEncodeFn>(ptr);
  }
  return fn;
}

}  // namespace lx

extern "C" {

// 1: the tensor-core kernel takes this shape (d = 128, an even number of query heads per KV head, 16-byte aligned strides).
int lx_attn_prefill_tc_supported(int nh, int nkv, int d, long long ldq, long long ldo) {
  return (d == 128 && nkv > 0 && nh % nkv == 0 && ((nh / nkv) % 2) == 0 && ldq % 8 == 0 && ldo % 8 == 0) ? 1 : 0;
}

// Same contract as lx_attn_prefill_alibi (64-query tiles listed by tile_seq / tile_q0), plus the number of tokens `T` of the q
// buffer and the number of blocks of the cache (bounds of the two tensor maps) and the status word.
int lx_attn_prefill_tc(const void* q, long long ldq, int T, const void* kv, int num_blocks, const int* block_tables, int max_blocks,
                       const int* cu_q, const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo,
                       int nh, int nkv, int d, int window, float scale, float softcap, const float* alibi, int* status, void* stream) {
  using namespace lx;
  if (num_tiles <= 0) return 0;
  if (!lx_attn_prefill_tc_supported(nh, nkv, d, ldq, ldo)) return -1;
  FaEncodeFn fn = fa_encode_fn();
  if (fn == nullptr) return -2;
  CUtensorMap tq, tkv;
  {
    cuuint64_t dims[2] = {(cuuint64_t)nh * kFaD, (cuuint64_t)T};
    cuuint64_t strides[1] = {(cuuint64_t)ldq * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)kFaQ};
    cuuint32_t es[2] = {1, 1};
    if (fn(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -3;
  }
  {
    cuuint64_t dims[5] = {(cuuint64_t)kFaD, (cuuint64_t)kFaPage, 2, (cuuint64_t)nkv, (cuuint64_t)num_blocks};
    cuuint64_t strides[4] = {(cuuint64_t)kFaD * 2, (cuuint64_t)kFaPage * kFaD * 2, (cuuint64_t)2 * kFaPage * kFaD * 2,
                             (cuuint64_t)nkv * 2 * kFaPage * kFaD * 2};
    cuuint32_t box[5] = {64, (cuuint32_t)kFaPage, 1, 1, 1};
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    if (fn(&tkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(kv), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return -4;
  }
  FaParams p{};
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.cu_q = cu_q; p.cache_lens = cache_lens;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.nh = nh; p.nkv = nkv; p.group = nh / nkv; p.window = window; p.scale = scale; p.softcap = softcap; p.alibi = alibi; p.status = status;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FaSmem::kTotal);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  launch_pdl(attn_prefill_tc_kernel, dim3(num_tiles, nh / 2), dim3(kFaThreads), (size_t)FaSmem::kTotal, reinterpret_cast<cudaStream_t>(stream),
             tq, tkv, p);
  return -(int)cudaGetLastError();
}

}  // extern "C"
