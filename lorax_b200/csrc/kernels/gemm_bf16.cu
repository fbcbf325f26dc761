// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands fed by TMA).
//
//   out[i, j] = sum_k A[i, k] * B[j, k]  (+ bias)          A: [a_rows, K]   B: [b_rows, K]   both K-contiguous
//
// One kernel serves every dense projection of the decoder (QKV, O, gate_up, down, lm_head), which the
// reference computes with cuBLAS through `torch.nn.functional.linear` (server/lorax_server/layers/linear.py:38).
// Both operands are "K-major", which is how activations [tokens, K] and nn.Linear weights [N, K] already sit in
// memory, so either can take the UMMA M side:
//   * prefill (many tokens):  A = activations, B = weights, 128 x 256 tiles, compute bound;
//   * decode (few tokens):    A = weights (128 output features per tile), B = activations (UMMA N = tokens
//     rounded up to 16), so the tensor core does no work for padding rows and each weight byte is read from
//     HBM exactly once.  Small grids are widened with split-K; the last CTA to finish a tile reduces the
//     fp32 partials in a fixed order (deterministic) and writes bf16.
//
// Structure: persistent CTAs of 6 warps.  Warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) and
// TMEM owner, warps 2..5 = epilogue (each warp reads its own 32-lane TMEM quadrant with tcgen05.ld).  A STAGES
// deep smem ring is guarded by full/empty mbarriers; the accumulator is double buffered in TMEM so the epilogue
// of tile i overlaps the main loop of tile i+1.
#include "common.cuh"

namespace lx {

constexpr int kBM = 128;   // UMMA M (rows of operand A per tile)
constexpr int kBK = 64;    // K per pipeline stage: 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int lx_gemm_max_tiles_const = 8192;

struct GemmParams {
  int a_rows, b_rows, K;
  int umma_n;                 // runtime UMMA N (multiple of 16, <= bn)
  int bn;                     // rows of operand B per tile (multiple of 16, <= the template's BN, which sizes smem and TMEM)
  __nv_bfloat16* out;
  long long ldo_a, ldo_b;     // out[i * ldo_a + j * ldo_b]
  const __nv_bfloat16* bias;  // optional, indexed by the feature dimension
  int bias_on_a;              // 1: bias[i] (weights are operand A), 0: bias[j]
  int split_k;
  float* ws;                  // split-K partials: [tile][split][128][BN] fp32
  int* counters;              // split-K arrival counters, one per tile, zero between launches
  int* status;                // [2] status word + detail
  int hint_a_first;           // 1: operand A is streamed once (weights) -> evict_first, B evict_last; 0: opposite
  float out_scale;            // multiplies the accumulator (logit scaling); 1.0 normally
  int b_fastest;              // tile order: 1 = B tile index fastest (CTAs running together share the A tile in L2)
  // Stream-K (used when split_k == 1): the first dp_tiles tiles are computed whole, one per CTA per wave; the K
  // loops of the remaining tiles are laid end to end and cut into sk_ctas equal ranges, so the last, partly
  // filled wave costs its share of a wave instead of a whole one.  dp_tiles == all tiles switches it off.
  int dp_tiles;
  int sk_ctas;
  // Multi-adapter LoRA delta added in the epilogue (lora_v == nullptr: none):
  //   out[t, n] += sum_j lora_v[t, part(n) * r + j] * B_cat(slot(t))[n, j],   r = slot_rank[slot(t)]
  // lora_v is the shrink result x A^T (fp32), B_cat [N, r] sits in the adapter arena at
  // slot_base[slot] + r * lora_unit_off and already carries the alpha / r scaling.
  const float* lora_v;
  int lora_ldv;
  const int* lora_tok_slot;            // [tokens] adapter slot per token, -1 = none
  const __nv_bfloat16* lora_arena;
  const long long* lora_slot_base;
  const int* lora_slot_rank;
  int lora_num_slots;
  long long lora_unit_off;
  int lora_n0, lora_n1;                // part boundaries along the feature dimension (q | k | v, gate | up)
  int tokens_on_a;                     // 1: tile rows are tokens (activations are operand A), 0: tile rows are features
};

// ---- LoRA epilogue ------------------------------------------------------------------------------------------
// The delta is added to NC accumulator columns at a time, rank in slices of 8 (16 bytes of B, two float4 of v).
// Every load address is computed without a branch (dead lanes read a valid dummy address and multiply by zero), so
// the loads of all NC columns are independent and the compiler can keep many in flight: the epilogue warps have no
// other warps to hide memory latency behind.
LX_DEVICE float lora_dot8(const uint4 b, const float4 v0, const float4 v1) {
  const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
  float acc = v0.x * b0.x;
  acc = fmaf(v0.y, b0.y, acc); acc = fmaf(v0.z, b1.x, acc); acc = fmaf(v0.w, b1.y, acc);
  acc = fmaf(v1.x, b2.x, acc); acc = fmaf(v1.y, b2.y, acc); acc = fmaf(v1.z, b3.x, acc); acc = fmaf(v1.w, b3.y, acc);
  return acc;
}

// Adapter of one token, resolved once: rank (0 = no adapter), where its B_cat of this projection group starts, its v row.
struct LoraTok {
  int r;
  const __nv_bfloat16* b;
  const float* v;
};
LX_DEVICE LoraTok lora_token(const GemmParams& p, int t, int num_tokens) {
  LoraTok k{0, p.lora_arena, p.lora_v};
  if (t < num_tokens) {
    const int s = p.lora_tok_slot[t];
    if (s >= 0 && s < p.lora_num_slots) {
      const int r = p.lora_slot_rank[s];
      const long long base = p.lora_slot_base[s];
      if (r > 0 && base >= 0) {
        k.r = r;
        k.b = p.lora_arena + base + (long long)r * p.lora_unit_off;
        k.v = p.lora_v + (long long)t * p.lora_ldv;
      }
    }
  }
  return k;
}

// acc[q] += delta(feature row i, token column j + q) for q < NC (weights-on-A orientation, NC <= 32).
// Lane q of the warp resolves token j + q and copies that token's slice of the shrink result into the warp's
// staging area, 16 ranks at a time; every lane then reads it back as broadcasts while its own B row (32 bytes per
// 16 ranks) comes straight from the arena, eight columns' loads issued before the first is used.
template <int NC>
LX_DEVICE void lora_add_token_columns(const GemmParams& p, float (&acc)[NC], int i, int j, int jend, float* stage) {
  const int lane = threadIdx.x & 31;
  const LoraTok tok = lora_token(p, j + lane, (lane < NC) ? jend : 0);
  const int rmax = __reduce_max_sync(0xffffffffu, tok.r);
  if (rmax == 0) return;
  const int part = i < p.lora_n0 ? 0 : (i < p.lora_n1 ? 1 : 2);
  const int part0 = __shfl_sync(0xffffffffu, part, 0);
  const bool part_uniform = __all_sync(0xffffffffu, part == part0);
  const bool row_ok = i < p.a_rows;
  constexpr int NB = NC < 8 ? NC : 8;
  for (int jc = 0; jc < rmax; jc += 16) {
    if (part_uniform) {
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        if (jc + 4 * h < tok.r) z = __ldg(reinterpret_cast<const float4*>(tok.v + part0 * tok.r + jc + 4 * h));
        *reinterpret_cast<float4*>(stage + lane * 16 + 4 * h) = z;
      }
      __syncwarp();
    }
#pragma unroll
    for (int q0 = 0; q0 < NC; q0 += NB) {
      uint4 b0[NB], b1[NB];
      int rq[NB];
#pragma unroll
      for (int u = 0; u < NB; ++u) {
        rq[u] = __shfl_sync(0xffffffffu, tok.r, q0 + u);
        const __nv_bfloat16* bq = reinterpret_cast<const __nv_bfloat16*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(tok.b), q0 + u));
        const __nv_bfloat16* row = bq + (long long)i * rq[u] + jc;
        b0[u] = __ldg(reinterpret_cast<const uint4*>((row_ok && jc < rq[u]) ? row : p.lora_arena));
        b1[u] = __ldg(reinterpret_cast<const uint4*>((row_ok && jc + 8 < rq[u]) ? row + 8 : p.lora_arena));
      }
#pragma unroll
      for (int u = 0; u < NB; ++u) {
        float4 v0, v1, v2, v3;
        if (part_uniform) {
          const float4* sv = reinterpret_cast<const float4*>(stage + (q0 + u) * 16);
          v0 = sv[0]; v1 = sv[1]; v2 = sv[2]; v3 = sv[3];
        } else {                  // a part boundary inside the warp's 32 features: every lane reads its own part
          const float* vq = reinterpret_cast<const float*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(tok.v), q0 + u));
          const float* vp = vq + part * rq[u] + jc;
          const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
          v0 = jc < rq[u] ? __ldg(reinterpret_cast<const float4*>(vp)) : zero;
          v1 = jc + 4 < rq[u] ? __ldg(reinterpret_cast<const float4*>(vp + 4)) : zero;
          v2 = jc + 8 < rq[u] ? __ldg(reinterpret_cast<const float4*>(vp + 8)) : zero;
          v3 = jc + 12 < rq[u] ? __ldg(reinterpret_cast<const float4*>(vp + 12)) : zero;
        }
        const float d0 = (row_ok && jc < rq[u]) ? lora_dot8(b0[u], v0, v1) : 0.f;
        const float d1 = (row_ok && jc + 8 < rq[u]) ? lora_dot8(b1[u], v2, v3) : 0.f;
        acc[q0 + u] += d0 + d1;
      }
    }
    __syncwarp();
  }
}

// acc[q] += delta(token row i, feature column j + q) for q < NC (tokens-on-A orientation): the thread's token is
// fixed, its B rows change with the column.  Plain loads; the serving paths use the other orientation.
template <int NC>
LX_DEVICE void lora_add_feature_columns(const GemmParams& p, float (&acc)[NC], int j, int jend, const LoraTok& mine) {
  const int rmax = __reduce_max_sync(0xffffffffu, mine.r);
  for (int jc = 0; jc < rmax; jc += 8) {
    const bool live_row = jc < mine.r;
#pragma unroll
    for (int q = 0; q < NC; ++q) {
      const int n = j + q;
      const bool live = live_row && n < jend;
      const int part = n < p.lora_n0 ? 0 : (n < p.lora_n1 ? 1 : 2);
      const __nv_bfloat16* bp = live ? mine.b + (long long)n * mine.r + jc : p.lora_arena;
      const float* vp = live ? mine.v + part * mine.r + jc : p.lora_v;
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(bp));
      const float4 v0 = __ldg(reinterpret_cast<const float4*>(vp));
      const float4 v1 = __ldg(reinterpret_cast<const float4*>(vp + 4));
      acc[q] += live ? lora_dot8(b, v0, v1) : 0.f;
    }
  }
}

// One unit of work of a CTA: k-blocks [kb0, kb1) of one output tile.  nparts == 0: the CTA owns the whole tile and
// writes bf16 directly.  Otherwise the fp32 partial goes to `part_off` (floats from ws), the arrival is counted in
// counters[counter], and the last of the nparts contributors sums partials red_base + i * red_stride
// (i = 0 .. nparts-1; the first one at red_first instead) in that fixed order.
struct GemmWork {
  int tile, kb0, kb1, nparts, counter;
  long long part_off, red_first, red_base, red_stride;
};

// Enumerates a CTA's work.  Producer, MMA issuer and epilogue warps each run their own copy in lockstep.
template <int BN>
struct GemmWorkIter {
  int num_tiles, kblocks, split_k, grid, cta, dp_tiles, sk_ctas;
  int i, phase;
  long long sk_units, u, u_begin, u_end;
  __device__ GemmWorkIter(const GemmParams& p, int num_tiles_, int kblocks_)
      : num_tiles(num_tiles_), kblocks(kblocks_), split_k(p.split_k), grid((int)gridDim.x), cta((int)blockIdx.x),
        dp_tiles(p.split_k > 1 ? 0 : p.dp_tiles), sk_ctas(p.sk_ctas), i(0), phase(0) {
    sk_units = (long long)(num_tiles - dp_tiles) * kblocks;
    u = u_begin = u_end = 0;
  }
  __device__ long long sk_start(int c) const { return sk_units * c / sk_ctas; }
  __device__ int sk_cta_of(long long unit) const { return (int)(((unit + 1) * sk_ctas - 1) / sk_units); }
  __device__ bool next(GemmWork& w) {
    constexpr long long kPart = (long long)BN * kBM;
    if (split_k > 1) {                       // classic split-K: every tile cut into split_k equal parts
      const int x = cta + i * grid;
      if (x >= num_tiles * split_k) return false;
      ++i;
      const int split = x % split_k;
      w.tile = x / split_k;
      w.kb0 = (int)((long long)kblocks * split / split_k);
      w.kb1 = (int)((long long)kblocks * (split + 1) / split_k);
      w.nparts = split_k;
      w.counter = w.tile;
      w.red_base = (long long)w.tile * split_k * kPart;
      w.red_first = w.red_base;
      w.red_stride = kPart;
      w.part_off = w.red_base + split * kPart;
      return true;
    }
    if (phase == 0) {
      const int t = cta + i * grid;
      if (t < dp_tiles) {
        ++i;
        w.tile = t; w.kb0 = 0; w.kb1 = kblocks; w.nparts = 0;
        return true;
      }
      phase = 1;
      if (cta < sk_ctas && sk_units > 0) {
        u_begin = u = sk_start(cta);
        u_end = sk_start(cta + 1);
      }
    }
    if (u >= u_end) return false;
    const int r = (int)(u / kblocks);
    const long long t0 = (long long)r * kblocks;
    w.tile = dp_tiles + r;
    w.kb0 = (int)(u - t0);
    const long long rem = u_end - u;
    w.kb1 = (rem >= kblocks - w.kb0) ? kblocks : w.kb0 + (int)rem;
    const bool first_seg = (u == u_begin);
    u += w.kb1 - w.kb0;
    if (w.kb0 == 0 && w.kb1 == kblocks) { w.nparts = 0; return true; }
    const int first = sk_cta_of(t0), last = sk_cta_of(t0 + kblocks - 1);
    w.nparts = last - first + 1;
    w.counter = r;
    w.part_off = (long long)(cta * 2 + (first_seg ? 0 : 1)) * kPart;
    w.red_base = (long long)(first * 2) * kPart;
    w.red_stride = 2 * kPart;
    w.red_first = w.red_base + (sk_start(first) < t0 ? kPart : 0);
    return true;
  }
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kLoraBytes = 4 * 32 * 16 * 4;   // per epilogue warp: 32 tokens x 16 ranks of the shrink result
  static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + kLoraBytes + 1024;  // +1024 for manual alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  pdl_trigger();
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* last_flag = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_base_slot + 2));
  float* lora_stage_all = reinterpret_cast<float*>(smem + STAGES * S::kStageBytes + S::kBarrierBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;

  const int tiles_a = (p.a_rows + kBM - 1) / kBM;
  const int tiles_b = (p.b_rows + p.bn - 1) / p.bn;
  const int num_tiles = tiles_a * tiles_b;
  const int kblocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tmem_full[s], 1);
      mbar_init(&tmem_empty[s], 4);
    }
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_wait();      // barriers, TMEM and descriptors are set up while the previous kernel drains; its data is read from here on

  // Work item w -> (tile, split).  Tiles are ordered with the A tile index fastest inside one B tile so that
  // CTAs running at the same time share the B operand through L2.
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_a = p.hint_a_first ? policy_evict_first() : policy_evict_last();
      const uint64_t pol_b = p.hint_a_first ? policy_evict_last() : policy_evict_first();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      GemmWorkIter<BN> it(p, num_tiles, kblocks);
      GemmWork w;
      while (ok && it.next(w)) {
        const int ta = p.b_fastest ? w.tile / tiles_b : w.tile % tiles_a;
        const int tb = p.b_fastest ? w.tile % tiles_b : w.tile / tiles_a;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kTimeoutEmptyBarrier, w.tile);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = tiles + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_expect_tx(&full_bar[stage], (uint32_t)(S::kABytes + p.bn * kBK * 2));
          tma_load_2d_hint(sa, &tmap_a, &full_bar[stage], kb * kBK, ta * kBM, pol_a);
          tma_load_2d_hint(sb, &tmap_b, &full_bar[stage], kb * kBK, tb * p.bn, pol_b);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kBM, (uint32_t)p.umma_n, kFmtBF16, kFmtBF16);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      GemmWorkIter<BN> it(p, num_tiles, kblocks);
      GemmWork w;
      while (ok && it.next(w)) {
        const int kb0 = w.kb0, kb1 = w.kb1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_flag)) {
          report_status(p.status, kTimeoutTmemEmpty, w.tile);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            report_status(p.status, kTimeoutFullBarrier, w.tile);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * S::kStageBytes);
          const uint64_t da = make_desc_k_sw128(sa);
          const uint64_t db = make_desc_k_sw128(sa + S::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            umma_f16_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);   // releases the smem stage when these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);       // accumulator complete
        acc_phase[acc] ^= 1;
        acc ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..5)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    GemmWorkIter<BN> it(p, num_tiles, kblocks);
    GemmWork w;
    while (it.next(w)) {
      const int ta = p.b_fastest ? w.tile / tiles_b : w.tile % tiles_a;
      const int tb = p.b_fastest ? w.tile % tiles_b : w.tile / tiles_a;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_flag)) {
        report_status(p.status, kTimeoutTmemFull, w.tile);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      acc_phase[acc] ^= 1;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      const int i = ta * kBM + row_in_tile;
      const int j0 = tb * p.bn;
      const int ncols = min(p.bn, p.umma_n);
      const int jend = min(p.b_rows, j0 + ncols);     // columns past it belong to the next tile (or to nobody)
      constexpr int CH = (BN >= 32) ? 32 : 16;
      float* lora_stage = lora_stage_all + quad * (32 * 16);
      LoraTok lora_mine{0, nullptr, nullptr};
      if (p.lora_v != nullptr && p.tokens_on_a) lora_mine = lora_token(p, i, p.a_rows);

      if (w.nparts == 0) {
#pragma unroll 1
        for (int c = 0; c < ncols; c += CH) {
          float v[CH];
          if constexpr (CH == 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = __uint_as_float(r[q]);
          } else {
            uint32_t r[16];
            tmem_ld_32x32b_x16(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 16; ++q) v[q] = __uint_as_float(r[q]);
          }
#pragma unroll
          for (int q = 0; q < CH; ++q) v[q] *= p.out_scale;
          if (p.lora_v != nullptr) {
            if (p.tokens_on_a) lora_add_feature_columns<CH>(p, v, j0 + c, jend, lora_mine);
            else lora_add_token_columns<CH>(p, v, i, j0 + c, jend, lora_stage);
          }
          if (i < p.a_rows) {
            const float bias_i = (p.bias != nullptr && p.bias_on_a) ? __bfloat162float(p.bias[i]) : 0.f;
            __nv_bfloat16* orow = p.out + (long long)i * p.ldo_a;
            const int j = j0 + c;
            if (p.ldo_b == 1 && j + CH <= jend && ((reinterpret_cast<uintptr_t>(orow + j) & 15) == 0)) {
              uint32_t pk[CH / 2];
#pragma unroll
              for (int q = 0; q < CH; q += 2) {
                float b0 = bias_i, b1 = bias_i;
                if (p.bias != nullptr && !p.bias_on_a) {
                  b0 = __bfloat162float(p.bias[j + q]);
                  b1 = __bfloat162float(p.bias[j + q + 1]);
                }
                pk[q / 2] = pack_bf16x2(v[q] + b0, v[q + 1] + b1);
              }
              uint4* dst = reinterpret_cast<uint4*>(orow + j);
#pragma unroll
              for (int q = 0; q < CH / 8; ++q) dst[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            } else {
#pragma unroll
              for (int q = 0; q < CH; ++q) {
                if (j + q < jend) {
                  float b = bias_i;
                  if (p.bias != nullptr && !p.bias_on_a) b = __bfloat162float(p.bias[j + q]);
                  orow[(long long)(j + q) * p.ldo_b] = __float2bfloat16(v[q] + b);
                }
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      } else {
        // ---- split-K: park the fp32 partial, count arrivals, the last CTA of the tile reduces.
        // Partial layout [split][column][128 rows]: for a fixed column the 32 lanes of a warp touch 32
        // consecutive floats, so both the parking stores and the reducer's loads are fully coalesced.
        float* __restrict__ wsp = p.ws + w.part_off + row_in_tile;
#pragma unroll 1
        for (int c = 0; c < ncols; c += CH) {
          if constexpr (CH == 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q) __stcg(wsp + (long long)(c + q) * kBM, __uint_as_float(r[q]));
          } else {
            uint32_t r[16];
            tmem_ld_32x32b_x16(taddr + c, r);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 16; ++q) __stcg(wsp + (long long)(c + q) * kBM, __uint_as_float(r[q]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int prev = atomicAdd(&p.counters[w.counter], 1);
          *last_flag = (prev == w.nparts - 1) ? 1 : 0;
          if (prev == w.nparts - 1) p.counters[w.counter] = 0;   // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool is_last = (*last_flag != 0);
        if (is_last) {
          __threadfence();
          const bool row_ok = i < p.a_rows;
          const float bias_i = (row_ok && p.bias != nullptr && p.bias_on_a) ? __bfloat162float(p.bias[i]) : 0.f;
          __nv_bfloat16* __restrict__ orow = p.out + (long long)i * p.ldo_a;
          const float* __restrict__ base = p.ws + w.red_base + row_in_tile;
          const float* __restrict__ base0 = p.ws + w.red_first + row_in_tile;
          const long long sstride = w.red_stride;
          constexpr int RC = 16;      // columns reduced together: RC * 4 independent loads in flight
#pragma unroll 1
          for (int c = 0; c < ncols; c += RC) {
            float acc8[RC];
#pragma unroll
            for (int q = 0; q < RC; ++q) acc8[q] = 0.f;
#pragma unroll 4
            for (int sp = 0; sp < w.nparts; ++sp) {
              float t[RC];
              const float* __restrict__ src = (sp == 0) ? base0 : base + sp * sstride;
#pragma unroll
              for (int q = 0; q < RC; ++q) t[q] = __ldcg(src + (long long)(c + q) * kBM);
#pragma unroll
              for (int q = 0; q < RC; ++q) acc8[q] += t[q];
            }
#pragma unroll
            for (int q = 0; q < RC; ++q) acc8[q] *= p.out_scale;
            if (p.lora_v != nullptr) {
              if (p.tokens_on_a) lora_add_feature_columns<RC>(p, acc8, j0 + c, jend, lora_mine);
              else lora_add_token_columns<RC>(p, acc8, i, j0 + c, jend, lora_stage);
            }
            if (row_ok) {
              const int j = j0 + c;
              if (p.ldo_b == 1 && j + RC <= jend && ((reinterpret_cast<uintptr_t>(orow + j) & 15) == 0)) {
                uint32_t pk[RC / 2];
#pragma unroll
                for (int q = 0; q < RC; q += 2) {
                  float b0 = bias_i, b1 = bias_i;
                  if (p.bias != nullptr && !p.bias_on_a) {
                    b0 = __bfloat162float(p.bias[j + q]);
                    b1 = __bfloat162float(p.bias[j + q + 1]);
                  }
                  pk[q / 2] = pack_bf16x2(acc8[q] + b0, acc8[q + 1] + b1);
                }
                uint4* dst = reinterpret_cast<uint4*>(orow + j);
#pragma unroll
                for (int q = 0; q < RC / 8; ++q) dst[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
              } else {
#pragma unroll
                for (int q = 0; q < RC; ++q) {
                  if (j + q < jend) {
                    float b = bias_i;
                    if (p.bias != nullptr && !p.bias_on_a) b = __bfloat162float(p.bias[j + q]);
                    orow[(long long)(j + q) * p.ldo_b] = __float2bfloat16(acc8[q] + b);
                  }
                }
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag is reused by the next tile
      }
      acc ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// 2-D K-major bf16 tensor map: dims {K, rows}, box {64, box_rows}, 128-byte swizzle, zero fill outside.
int make_tmap_bf16_kmajor(CUtensorMap* out, const void* base, uint64_t rows, uint64_t K, uint64_t row_stride_elems,
                          uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  // the shared-memory opt-in is a per-device attribute: one flag per device ordinal
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  launch_pdl(gemm_bf16_tcgen05_kernel<BN, STAGES>, dim3(grid), dim3(kGemmThreads), (size_t)S::kTotal, stream, ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

// ---- planning -----------------------------------------------------------------------------------------------
// Times in nanoseconds for one SM.  A tile streams (128 + bn) * 2 * K bytes into shared memory (about 95 B/ns per SM
// when all SMs pull from L2 and HBM together) and issues 128 * bn * K MACs (about 11 TFLOP/s per SM); the slower of
// the two bounds it.  Every unit of work pays a fixed ramp, a stream-K partial pays its fp32 round trip through
// L2 and the last contributor pays the sum.  Constants fitted to sweeps on B200.
constexpr double kFillBytesPerNs = 95.0;
constexpr double kFlopPerNs = 11000.0;
constexpr double kTileFixedNs = 2500.0;

struct GemmPlan {
  int bn, split, dp_tiles, sk_ctas, grid;
  double cost;
};

static int template_bn(int bn) { return bn <= 16 ? 16 : bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256; }

// Decide how the last, partly filled wave of `tiles` tiles is computed.  sk_policy: 0 = by cost, 1 = never
// stream-K, 2 = stream-K whenever there is a remainder.
static GemmPlan plan_tiles(int tiles, int kblocks, int K, int bn, int num_sms, long long ws_bytes, bool have_counters, int sk_policy) {
  GemmPlan pl{};
  pl.bn = bn;
  pl.split = 1;
  pl.grid = tiles < num_sms ? tiles : num_sms;
  const int G = pl.grid;
  const int full_waves = tiles / G, R = tiles % G == 0 ? 0 : tiles - full_waves * G;
  const double fill = (double)(kBM + bn) * 2.0 * K / kFillBytesPerNs;
  const double mma = 2.0 * kBM * bn * (double)K / kFlopPerNs;
  const double t_tile = (fill > mma ? fill : mma) + kTileFixedNs;
  pl.dp_tiles = tiles;
  pl.sk_ctas = 0;
  pl.cost = (double)(full_waves + (R ? 1 : 0)) * t_tile;
  // a grid smaller than the GPU is all remainder: widen it to every SM
  const int rem = tiles < num_sms ? tiles : R;
  const int dp = tiles < num_sms ? 0 : full_waves * G;
  if (rem == 0 || sk_policy == 1 || !have_counters) return pl;
  // By cost, stream-K is only offered to grids smaller than the GPU with token tiles up to 128: there it replaces
  // the classic K split.  For larger problems the fp32 round trip of the partials costs more than the idle SMs.
  if (sk_policy == 0 && (dp != 0 || bn > 128)) return pl;
  const long long units = (long long)rem * kblocks;
  long long ctas = num_sms;
  if (ctas > units / 2) ctas = units / 2;
  if (ctas > 15ll * rem) ctas = 15ll * rem;
  const long long per_cta = 2ll * kBM * template_bn(bn) * 4;
  if (ctas * per_cta > ws_bytes) ctas = ws_bytes / per_cta;
  if (ctas < 2 || ctas <= rem) return pl;      // nothing to gain over whole tiles
  const double L = (double)units / (double)ctas;                     // k-blocks per CTA
  const double nparts = (double)kblocks / L + 1.0;
  const double part = (double)kBM * bn * 4.0;
  // measured: a partial costs about 1 ns per 5 bytes end to end (store, fence, arrival, the last CTA's sum), whatever the part count
  (void)nparts;
  const double sk_cost = (double)(dp ? full_waves : 0) * t_tile + (t_tile - kTileFixedNs) * L / kblocks + kTileFixedNs + part / 5.0 + 1500.0;
  if (sk_policy == 2 || sk_cost < pl.cost) {
    pl.dp_tiles = dp;
    pl.sk_ctas = (int)ctas;
    pl.grid = dp ? num_sms : (int)ctas;
    pl.cost = sk_cost;
  }
  return pl;
}

// Weights-on-M path: pick the token tile (UMMA N, any multiple of 16 up to 256).  Few tokens -> one token tile; many
// tokens -> the tile count that wastes the fewest SM slots (the weight tile is re-read from L2 by the CTAs that
// run next to each other).
static GemmPlan choose_plan_swap(int T, int N, int K, int num_sms, long long ws_bytes, bool have_counters, int force_split, int force_bn,
                                 int sk_policy) {
  const int tiles_a = (N + kBM - 1) / kBM;
  const int kblocks = (K + kBK - 1) / kBK;
  const int t16 = (T + 15) / 16 * 16;
  int bn_full = t16 < 256 ? t16 : 256;
  const bool bn_forced = (force_bn >= 16 && force_bn <= 256 && force_bn % 16 == 0);
  if (bn_forced && force_bn < bn_full) bn_full = force_bn;
  if (force_split > 0) {            // tests and the no-allocation entry ask for an exact classic split on the full token tile
    int s = force_split > kblocks ? kblocks : force_split;
    const int tt = (T + bn_full - 1) / bn_full;
    if (s > 1 && ((long long)tiles_a * tt * s * kBM * template_bn(bn_full) * 4 > ws_bytes || tiles_a * tt > lx_gemm_max_tiles_const || !have_counters)) s = 1;
    GemmPlan pl{};
    pl.bn = bn_full; pl.split = s; pl.dp_tiles = tiles_a * tt; pl.sk_ctas = 0;
    const int work = tiles_a * tt * s;
    pl.grid = work < num_sms ? work : num_sms;
    return pl;
  }
  GemmPlan best{};
  best.cost = 1e30;
  for (int bn = bn_full; bn >= 16; bn -= 16) {
    const int ttiles = (T + bn - 1) / bn;
    GemmPlan pl = plan_tiles(tiles_a * ttiles, kblocks, K, bn, num_sms, ws_bytes, have_counters, sk_policy);
    if (pl.cost < best.cost) best = pl;
    if (bn_forced) break;
  }
  return best;
}

}  // namespace lx

extern "C" {

// Workspace sizes the caller must provide for split-K (bytes).
long long lx_gemm_ws_bytes() { return 64ll << 20; }
int lx_gemm_max_tiles() { return 8192; }

struct LxLoraEpilogue {
  const float* v;               // [T, ldv] shrink result
  int ldv;
  const int* tok_slot;          // [T]
  const void* arena;
  const long long* slot_base;
  const int* slot_rank;
  int num_slots;
  long long unit_off;           // B_cat of this projection group sits at slot_base + rank * unit_off
  int n0, n1;                   // part boundaries (N when the group has fewer parts)
};

static int gemm_impl(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                     long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                     int* status, int num_sms, int mode, int force_split, const LxLoraEpilogue* lora, void* stream_) {
  using namespace lx;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return -1000;
  const int sk_policy = (mode >> 8) & 3;      // 0 by cost, 1 whole tiles only, 2 stream-K whenever a wave is partly filled
  mode &= 0xff;
  const bool have_counters = (ws != nullptr && counters != nullptr);
  const long long usable_ws = have_counters ? ws_bytes : 0;
  GemmPlan pl{};
  GemmParams p{};
  p.K = K;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ws = reinterpret_cast<float*>(ws);
  p.counters = counters;
  p.status = status;
  p.out_scale = out_scale;
  p.split_k = 1;
  CUtensorMap ta, tb;
  int bn;
  const bool has_lora = (lora != nullptr && lora->v != nullptr);
  const int force_bn = force_split >> 16;
  const int kblocks_all = (K + kBK - 1) / kBK;
  // Tokens on the M side: the feature tile (UMMA N) whose tile count wastes the fewest SM slots in the last wave;
  // 32-wide steps keep the epilogue's 16-byte stores whole.
  GemmPlan pl_tok{};
  pl_tok.cost = 1e30;
  {
    const int tiles_t = (T + kBM - 1) / kBM;
    for (int cand = 256; cand >= 64; cand -= 32) {
      if (force_bn >= 32 && force_bn <= 256 && force_bn % 32 == 0 && cand != force_bn) continue;
      GemmPlan c = plan_tiles(tiles_t * ((N + cand - 1) / cand), kblocks_all, K, cand, num_sms, usable_ws, have_counters, sk_policy);
      if (c.cost < pl_tok.cost) pl_tok = c;
    }
    if (pl_tok.cost >= 1e30) pl_tok = plan_tiles(tiles_t * ((N + 255) / 256), kblocks_all, K, 256, num_sms, usable_ws, have_counters, sk_policy);
  }
  // Orientation.  Up to 128 tokens the weights take the M side (no padded MMA rows, the token tile is the small
  // operand).  Above that both plans are costed; the weights-on-M epilogue writes 2 bytes per thread and store, which
  // measures about 15 % slower at equal tiling.  The LoRA epilogue's fast path is written for weights on M.
  bool swap;
  GemmPlan pl_swap{};
  if (mode == 1 || (mode == 0 && (T <= 128 || (has_lora && T <= 2048)))) {
    swap = true;
  } else if (mode == 2 || T > 2048) {
    swap = false;
  } else {
    pl_swap = choose_plan_swap(T, N, K, num_sms, usable_ws, have_counters, force_split & 0xffff, force_bn, sk_policy);
    swap = pl_swap.cost * 1.15 < pl_tok.cost;
  }
  if (swap) {
    p.a_rows = N; p.b_rows = T;
    p.ldo_a = 1; p.ldo_b = ldo;
    p.bias_on_a = 1;
    p.hint_a_first = 1;
    p.b_fastest = 1;          // token tiles of one weight tile run side by side: the weight tile leaves HBM once
    pl = choose_plan_swap(T, N, K, num_sms, usable_ws, have_counters, force_split & 0xffff, force_split >> 16, sk_policy);
    bn = pl.bn;
    p.umma_n = bn;
    if (make_tmap_bf16_kmajor(&ta, w, N, K, ldw, kBM)) return -1002;
    if (make_tmap_bf16_kmajor(&tb, x, T, K, ldx, bn)) return -1003;
  } else {
    pl = pl_tok;
    bn = pl.bn;
    p.a_rows = T; p.b_rows = N;
    p.umma_n = bn;
    p.ldo_a = ldo; p.ldo_b = 1;
    p.bias_on_a = 0;
    p.hint_a_first = 0;
    p.b_fastest = 0;
    if (make_tmap_bf16_kmajor(&ta, x, T, K, ldx, kBM)) return -1002;
    if (make_tmap_bf16_kmajor(&tb, w, N, K, ldw, bn)) return -1003;
  }
  p.bn = bn;
  p.split_k = pl.split;
  p.dp_tiles = pl.dp_tiles;
  p.sk_ctas = pl.sk_ctas;
  p.tokens_on_a = swap ? 0 : 1;
  if (lora != nullptr && lora->v != nullptr) {
    p.lora_v = lora->v; p.lora_ldv = lora->ldv; p.lora_tok_slot = lora->tok_slot;
    p.lora_arena = reinterpret_cast<const __nv_bfloat16*>(lora->arena);
    p.lora_slot_base = lora->slot_base; p.lora_slot_rank = lora->slot_rank; p.lora_num_slots = lora->num_slots;
    p.lora_unit_off = lora->unit_off; p.lora_n0 = lora->n0; p.lora_n1 = lora->n1;
  }
  switch (template_bn(bn)) {
    case 16:  return launch_gemm<16, 8>(ta, tb, p, pl.grid, stream);
    case 32:  return launch_gemm<32, 8>(ta, tb, p, pl.grid, stream);
    case 64:  return launch_gemm<64, 8>(ta, tb, p, pl.grid, stream);
    case 128: return launch_gemm<128, 6>(ta, tb, p, pl.grid, stream);
    default:  return launch_gemm<256, 4>(ta, tb, p, pl.grid, stream);
  }
}

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N]).  `ldx`, `ldw`, `ldo` are row strides in elements.
// mode: low byte 0 = choose, 1 = force weights on the M side (small T), 2 = force activations on the M side; bits 8..9 the
// stream-K policy (0 by cost, 1 whole tiles only, 2 stream-K whenever a wave is partly filled).
// force_split: low 16 bits an exact classic K split, high 16 bits a forced token tile.
// Returns 0 or a negative error; device-side timeouts are reported through `status` (2 ints, zeroed by the caller).
// The plan the weights-on-M path would use for a shape: out5 = {token tile, classic split, whole tiles, stream-K CTAs, grid}.
int lx_gemm_plan(int T, int N, int K, int num_sms, long long ws_bytes, int force_split, int sk_policy, int* out5) {
  lx::GemmPlan pl = lx::choose_plan_swap(T, N, K, num_sms, ws_bytes, ws_bytes > 0, force_split & 0xffff, force_split >> 16, sk_policy);
  out5[0] = pl.bn; out5[1] = pl.split; out5[2] = pl.dp_tiles; out5[3] = pl.sk_ctas; out5[4] = pl.grid;
  return 0;
}

int lx_gemm_bf16(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                 long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                 int* status, int num_sms, int mode, int force_split, void* stream_) {
  return gemm_impl(x, w, out, bias, T, N, K, ldx, ldw, ldo, out_scale, ws, ws_bytes, counters, status, num_sms, mode, force_split,
                   nullptr, stream_);
}

// The same GEMM with the multi-adapter LoRA delta added in the epilogue: one kernel replaces the base GEMM plus the
// expand kernel of the reference (server/lorax_server/utils/layers.py:114-164 runs them as separate launches and the
// expand reads and rewrites the whole output).
int lx_gemm_bf16_lora(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                      long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                      int* status, int num_sms, int mode, int force_split, const float* lora_v, int lora_ldv,
                      const int* tok_slot, const void* arena, const long long* slot_base, const int* slot_rank, int num_slots,
                      long long unit_off, int n0, int n1, void* stream_) {
  LxLoraEpilogue l{lora_v, lora_ldv, tok_slot, arena, slot_base, slot_rank, num_slots, unit_off, n0, n1};
  return gemm_impl(x, w, out, bias, T, N, K, ldx, ldw, ldo, out_scale, ws, ws_bytes, counters, status, num_sms, mode, force_split,
                   &l, stream_);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in lx_noalloc.h).
//
// The split-K path above needs scratch: fp32 partial tiles plus one arrival counter per output tile.  The
// regular entry point takes that scratch from its caller.  Some callers cannot provide any: code that runs
// inside a stream capture, a real-time or safety-partitioned host that forbids cudaMalloc after start-up, a
// plugin living in another framework's process whose allocator it must not touch.  For them the same kernel is
// offered with its scratch in a fixed array that is part of this library's image.
//
// Limits, because the array is static: it is kNoAllocPartialBytes + kNoAllocCounters*4 + 16 bytes on EVERY
// GPU that loads this library, from load until the process exits.  Problems whose split-K partials would not
// fit are rejected (or, with split_k = 0, run with a smaller split that fits, down to no split at all).
// All calls share the one array and it keeps what the previous call left: the counters are cleared on the
// stream before every launch, the partials are fully overwritten before they are read.  Two calls that
// overlap on the GPU (different streams, or different host threads without ordering) would race on it.
// ------------------------------------------------------------------------------------------------
namespace lx {

constexpr long long kNoAllocPartialBytes = 8ll << 20;   // 8 MiB of fp32 partial tiles
constexpr int kNoAllocCounters = 1024;                  // one per 128-row output tile
constexpr int kNoAllocMaxDevices = 64;

struct NoAllocScratch {
  float partials[kNoAllocPartialBytes / 4];
  int counters[kNoAllocCounters];
  int status[4];
};

// In host code this name is only a handle for cudaGetSymbolAddress; it is NOT a device pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

// Device address of the array, per device, resolved on the first call made while that device is current.
static NoAllocScratch* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};

static int noalloc_scratch_for_current_device(NoAllocScratch** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return -2001;
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) return -2002;
    g_noalloc_ptr[dev] = reinterpret_cast<NoAllocScratch*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace lx

extern "C" {

long long lx_gemm_bf16_noalloc_scratch_bytes() { return (long long)sizeof(lx::NoAllocScratch); }
int lx_gemm_bf16_noalloc_max_tokens() { return 256; }

const char* lx_gemm_bf16_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -2001: return "no current CUDA device (or device ordinal >= 64)";
    case -2002: return "cudaGetSymbolAddress failed for the static scratch array";
    case -2003: return "T exceeds the 256-token maximum of the no-allocation entry point";
    case -2004: return "N needs more than 1024 output tiles (N > 131072): beyond the static counter array";
    case -2005: return "requested split_k does not fit the 8 MiB static scratch for this N and T";
    case -2006: return "K must be positive; K, ldx and ldw must be multiples of 8 elements (16-byte TMA alignment)";
    case -2007: return "clearing the arrival counters failed";
    default: return "launch or tensor-map error (negative CUDA / driver code)";
  }
}

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N]), T <= 256, same math and the same kernel as lx_gemm_bf16 in its
// weights-on-M mode.  split_k: 0 = largest power of two that fits the static scratch and fills the GPU,
// otherwise the exact split to use (rejected with -2005 when its partials do not fit).
//
// The first call made on a device resolves the device address of the static array (cudaGetSymbolAddress) and
// sets the kernel's shared-memory attribute; make that first call outside any stream capture.  No cudaMalloc,
// cudaFree or other allocating routine is called, on any call.
int lx_gemm_bf16_noalloc(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                         long long ldw, long long ldo, int split_k, void* stream_) {
  using namespace lx;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || N <= 0) return 0;
  if (T > 256) return -2003;
  if (K <= 0 || (K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0) return -2006;
  NoAllocScratch* sc = nullptr;
  if (int rc = noalloc_scratch_for_current_device(&sc)) return rc;
  const int tiles = (N + kBM - 1) / kBM;
  if (tiles > kNoAllocCounters) return -2004;
  const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  const int kblocks = (K + kBK - 1) / kBK;
  const long long per_split = (long long)tiles * kBM * bn * 4;
  int num_sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  if (num_sms <= 0) num_sms = 148;
  int split = 1;
  if (split_k > 0) {
    split = split_k > kblocks ? kblocks : split_k;
    if (split > 1 && per_split * split > kNoAllocPartialBytes) return -2005;
  } else {
    while (tiles * split < num_sms && kblocks / (split * 2) >= 4 && split < 16 && per_split * split * 2 <= kNoAllocPartialBytes) split *= 2;
  }
  GemmParams p{};
  p.K = K;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ws = sc->partials;
  p.counters = sc->counters;
  p.status = sc->status;
  p.out_scale = 1.f;
  p.split_k = split;
  p.bn = bn;
  p.dp_tiles = tiles;          // whole tiles or the classic split only: stream-K scratch would not fit the static array
  p.sk_ctas = 0;
  p.b_fastest = 1;
  p.a_rows = N; p.b_rows = T;
  p.umma_n = (T + 15) / 16 * 16;
  p.ldo_a = 1; p.ldo_b = ldo;
  p.bias_on_a = 1;
  p.hint_a_first = 1;
  CUtensorMap ta, tb;
  if (make_tmap_bf16_kmajor(&ta, w, N, K, ldw, kBM)) return -1002;
  if (make_tmap_bf16_kmajor(&tb, x, T, K, ldx, bn)) return -1003;
  // The array keeps the previous call's contents: counters (and the status words) must start at zero.
  if (cudaMemsetAsync(sc->counters, 0, sizeof(int) * (kNoAllocCounters + 4), stream) != cudaSuccess) return -2007;
  const int work = tiles * split;
  const int grid = work < num_sms ? work : num_sms;
  switch (bn) {
    case 16:  return launch_gemm<16, 8>(ta, tb, p, grid, stream);
    case 32:  return launch_gemm<32, 8>(ta, tb, p, grid, stream);
    case 64:  return launch_gemm<64, 8>(ta, tb, p, grid, stream);
    case 128: return launch_gemm<128, 6>(ta, tb, p, grid, stream);
    default:  return launch_gemm<256, 4>(ta, tb, p, grid, stream);
  }
}

// Copies the two status words of the last launch on the current device to host memory.  The copy is queued on `stream`
// (pass the stream the GEMM was launched on, non-blocking streams included) and the call returns when it has completed.
// 0 in out2[0] means every bounded wait inside the kernel completed.
int lx_gemm_bf16_noalloc_status(int* out2, void* stream_) {
  using namespace lx;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  NoAllocScratch* sc = nullptr;
  if (int rc = noalloc_scratch_for_current_device(&sc)) return rc;
  cudaError_t e = cudaMemcpyAsync(out2, sc->status, 2 * sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return -(int)e;
}

}  // extern "C"
