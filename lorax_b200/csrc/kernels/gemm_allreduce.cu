// Row-parallel GEMM fused with its all-reduce over NVLink peer memory, in ONE kernel (decode-sized batches).
//
//   out[T, N] = sum over ranks r of  x_r[T, K_r] @ W_r[N, K_r]^T   (+ addend_r[T, N])  (+ bias)
//
// This is the tensor-parallel O / down projection.  The reference runs cuBLAS and then an NCCL all-reduce of the
// whole [T, N] activation (server/lorax_server/utils/layers.py:329-374), one kernel plus one collective launch per
// projection; here the collective is decomposed into reduce-scatter + all-gather and overlapped tile by tile:
//
//   phase A  every rank computes its partial product tile by tile on tcgen05 (weights on the UMMA M side, tokens
//            on N, accumulator in TMEM) and stores each fp32 partial tile straight from registers into the
//            receive buffer of the tile's OWNER rank (tile t belongs to rank t % world) with peer stores over
//            NVLink, then bumps the owner's arrival counter with a system-scope atomic;
//   phase B  the owner waits for `world` arrivals, adds the partials in rank order (deterministic), adds the bias,
//            rounds to bf16 and writes the finished slice into the output buffer of EVERY rank (the all-gather),
//            then bumps each rank's completion counter;
//   phase C  a rank leaves the kernel when its completion counter shows that all of its output has landed.
//
// Small batches (<= 64 tokens) use a one-hop variant of the same kernel: every rank stores its partial tiles into
// every rank's receive buffer and every rank reduces all tiles itself.  That moves `world` times more bytes, which is
// irrelevant at this size, and removes the second NVLink round trip, which is what decode latency is made of.
//
// `addend` carries this rank's partial LoRA delta (x_r A_r^T) B^T, so the LoRA intermediate is reduced by the same
// reduce-scatter and no separate collective is needed for it.
//
// All buffers live in a symmetric allocation (same layout on every rank, peer pointers in `peers`).  Counters only
// grow; each rank keeps the value every counter must reach in a local target table that the last CTA of a launch
// advances by that launch's contribution, so a launch needs no host-side sequence number and can be replayed from a
// CUDA graph with any mix of shapes (all ranks issue the same sequence of launches).  Every wait is bounded: on expiry the kernel records where it gave up and
// returns.  No TMA multicast is used anywhere; remote memory is only touched with plain stores and atomics.
#include "common.cuh"

namespace lx {

constexpr int kArBM = 128;
constexpr int kArBK = 64;
constexpr int kArThreads = 192;
constexpr int kArMaxRanks = 8;
constexpr int kArMaxTokens = 256;
constexpr int kArMaxSlots = 16;       // partial-sum slots per owned tile: world * K-splits
constexpr int kArTokChunkOne = 8;      // tokens per phase-B work item, one-hop mode
constexpr int kArTokChunkTwo = 32;     // ... two-hop mode (fewer, fatter items: each one ends with a system fence)
constexpr int kArOneShotTokens = 64;   // batches up to this size use the one-hop variant

// Layout of the symmetric communication buffer (identical on every rank).
struct ArLayout {
  long long recv_off;      // float  [kArMaxSlots][tiles_owned_max][kArMaxTokens][128]   slot = rank * ksplit + split
  long long out_off;       // bf16   [kArMaxTokens][N_max]
  long long arrived_off;   // int    [tiles_max]
  long long ctrl_off;      // int    [8]: 0 done, 2 cta_done (3 argmax arrivals, 5 argmax cta_done)
  long long target_off;    // int    [tiles_max + 2]: running targets of arrived[t], of `done`, of the argmax arrivals
  int tiles_owned_max;
  int tiles_max;
  int n_max;
};

struct ArParams {
  unsigned char* peers[kArMaxRanks];   // base of the symmetric buffer on every rank (peers[rank] is local)
  ArLayout lay;
  int rank, world;
  int T, N, K;
  int umma_n;
  int ttiles;                          // token tiles of BN tokens per feature tile (phase A parallelism)
  int ksplit;                          // K splits per (feature tile, token tile): their partials are summed by the owner too
  int oneshot;                         // 1: partials go to EVERY rank and every rank reduces all tiles (one NVLink hop)
  int tok_cap, tiles_cap;              // strides of the receive buffer in this mode
  const __nv_bfloat16* bias;
  const __nv_bfloat16* addend;         // optional [T, lda] local partial to add before the reduction
  long long lda;
  int* status;
  unsigned long long budget_ns;        // how long a wait for another GPU lasts before the kernel gives up
};

LX_DEVICE int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
LX_DEVICE void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded spin until *p >= target (signed difference, counters wrap safely).  Returns false on expiry.
LX_DEVICE int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Polls with relaxed loads and pays for one acquire fence when the value has arrived.
LX_DEVICE bool wait_counter(const int* p, int target, int* status, int where, unsigned long long budget_ns) {
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while (true) {
    if (ld_relaxed_sys(p) - target >= 0) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      return true;
    }
    if ((++polls & 1023u) == 0) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) { report_status(status, kTimeoutPeerFlag, where); return false; }
    }
  }
}

template <int BN, int STAGES>
struct ArSmem {
  static constexpr int kABytes = kArBM * kArBK * 2;
  static constexpr int kBBytes = BN * kArBK * 2;
  static constexpr int kStage = kABytes + kBBytes;
  static constexpr int kTotal = STAGES * kStage + 256 + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kArThreads, 1)
gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const ArParams p) {
  using S = ArSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStage);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kCols = 2 * BN < 32 ? 32 : 2 * BN;

  unsigned char* local = p.peers[p.rank];
  int* ctrl = reinterpret_cast<int*>(local + p.lay.ctrl_off);
  int* targets = reinterpret_cast<int*>(local + p.lay.target_off);
  const int num_tiles = (p.N + kArBM - 1) / kArBM;
  const int kblocks = (p.K + kArBK - 1) / kArBK;
  const int tok_chunk = p.oneshot ? kArTokChunkOne : kArTokChunkTwo;
  const int n_chunks = (p.T + tok_chunk - 1) / tok_chunk;
  const int per_tile = p.ttiles * p.ksplit;
  const int num_units = num_tiles * per_tile;      // phase A work: (feature tile, token tile, K split)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tmem_full[s], 1); mbar_init(&tmem_empty[s], 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u / per_tile, j = (u % per_tile) / p.ksplit, sp = u % p.ksplit;
        const int kb0 = (int)((long long)kblocks * sp / p.ksplit), kb1 = (int)((long long)kblocks * (sp + 1) / p.ksplit);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { report_status(p.status, kTimeoutEmptyBarrier, t); *abort_flag = 1; ok = false; break; }
          uint8_t* sa = smem + stage * S::kStage;
          mbar_expect_tx(&full_bar[stage], S::kStage);
          tma_load_2d_hint(sa, &tmap_w, &full_bar[stage], kb * kArBK, t * kArBM, pol_w);
          tma_load_2d_hint(sa + S::kABytes, &tmap_x, &full_bar[stage], kb * kArBK, j * BN, pol_x);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kArBM, (uint32_t)p.umma_n, kFmtBF16, kFmtBF16);
      int stage = 0; uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      for (int t = blockIdx.x; t < num_units && ok; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_flag)) { report_status(p.status, kTimeoutTmemEmpty, t); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        const int sp = t % p.ksplit;
        const int kb0 = (int)((long long)kblocks * sp / p.ksplit), kb1 = (int)((long long)kblocks * (sp + 1) / p.ksplit);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { report_status(p.status, kTimeoutFullBarrier, t); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStage);
          const uint64_t da = make_desc_k_sw128(sa), db = make_desc_k_sw128(sa + S::kABytes);
#pragma unroll
          for (int k = 0; k < kArBK / 16; ++k) umma_f16_ss(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&tmem_full[acc]);
        acc_phase[acc] ^= 1;
        acc ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ================================================================== epilogue warps: phases A-store, B, C
    const int quad = warp & 3;
    const int f = quad * 32 + lane;                     // feature inside the tile
    const int et = threadIdx.x - 64;                    // 0..127
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    // ---- phase A: ship partial tiles to their owners
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
      const int t = u / per_tile, tok_base = ((u % per_tile) / p.ksplit) * BN, sp = u % p.ksplit;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_flag)) { report_status(p.status, kTimeoutTmemFull, t); *abort_flag = 1; ok = false; break; }
      tc_fence_after();
      acc_phase[acc] ^= 1;
      const int owner = t % p.world, t_local = p.oneshot ? t : t / p.world;
      const long long slot_off = (((long long)(p.rank * p.ksplit + sp) * p.tiles_cap + t_local) * p.tok_cap) * kArBM + f;
      float* dst = reinterpret_cast<float*>(p.peers[owner] + p.lay.recv_off) + slot_off;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      const int n = t * kArBM + f;
      constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < p.umma_n; c += CH) {
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
        for (int q = 0; q < CH; ++q) {
          const int tok = tok_base + c + q;
          if (tok < p.T) {
            float val = v[q];
            if (p.addend != nullptr && sp == 0 && n < p.N) val += __bfloat162float(p.addend[(long long)tok * p.lda + n]);
            if (!p.oneshot) {
              dst[(long long)tok * kArBM] = val;         // peer store: 32 lanes -> 128 contiguous bytes
            } else {
#pragma unroll
              for (int r = 0; r < kArMaxRanks; ++r)
                if (r < p.world) reinterpret_cast<float*>(p.peers[r] + p.lay.recv_off)[slot_off + (long long)tok * kArBM] = val;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      // the barrier orders every thread's peer stores before the signalling threads; their release-at-system-scope
      // atomic is cumulative, so the stores are visible to whoever observes the count
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!p.oneshot) {
        if (et == 0) red_release_sys_add(reinterpret_cast<int*>(p.peers[owner] + p.lay.arrived_off) + t, 1);
      } else if (et < p.world) {
        red_release_sys_add(reinterpret_cast<int*>(p.peers[et] + p.lay.arrived_off) + t, 1);
      }
      acc ^= 1;
    }
    // ---- phase B: reduce the tiles this rank owns and broadcast the result
    const int n_owned = p.oneshot ? num_tiles : (num_tiles - p.rank + p.world - 1) / p.world;
    const int items = n_owned * n_chunks;
    const float* recv = reinterpret_cast<const float*>(local + p.lay.recv_off);
    const int* arrived = reinterpret_cast<const int*>(local + p.lay.arrived_off);
    for (int it = blockIdx.x; it < items && ok; it += gridDim.x) {
      const int t_local = it / n_chunks, chunk = it % n_chunks;
      const int t = p.oneshot ? t_local : t_local * p.world + p.rank;
      if (et == 0) {
        if (!wait_counter(arrived + t, targets[t] + p.world * per_tile, p.status, 1000 + t, p.budget_ns)) *abort_flag = 1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) { ok = false; break; }
      const int n = t * kArBM + f;
      const float b = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
      const int tok0 = chunk * tok_chunk, tok1 = min(tok0 + tok_chunk, p.T);
      for (int tok = tok0; tok < tok1; tok += 4) {
        float s[4] = {b, b, b, b};
#pragma unroll
        for (int r = 0; r < kArMaxSlots; ++r) {
          if (r < p.world * p.ksplit) {
            const float* src = recv + (((long long)r * p.tiles_cap + t_local) * p.tok_cap + tok) * kArBM + f;
#pragma unroll
            for (int q = 0; q < 4; ++q) if (tok + q < tok1) s[q] += __ldcg(src + (long long)q * kArBM);
          }
        }
        if (n < p.N && p.oneshot) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(local + p.lay.out_off) + n;
#pragma unroll
          for (int q = 0; q < 4; ++q) if (tok + q < tok1) o[(long long)(tok + q) * p.lay.n_max] = __float2bfloat16(s[q]);
        } else if (n < p.N) {
#pragma unroll
          for (int r = 0; r < kArMaxRanks; ++r) {
            if (r < p.world) {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.peers[r] + p.lay.out_off) + n;
#pragma unroll
              for (int q = 0; q < 4; ++q) if (tok + q < tok1) o[(long long)(tok + q) * p.lay.n_max] = __float2bfloat16(s[q]);
            }
          }
        }
      }
      if (!p.oneshot) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et < p.world) red_release_sys_add(reinterpret_cast<int*>(p.peers[et] + p.lay.ctrl_off), 1);
      }
    }
    // ---- phase C: my whole output has been written by its owners (not needed when every rank reduced for itself)
    if (et == 0 && ok && !p.oneshot) {
      if (!wait_counter(ctrl, targets[p.lay.tiles_max] + num_tiles * n_chunks, p.status, 2000, p.budget_ns)) *abort_flag = 1;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kCols); }
  // the last CTA of the launch advances the epoch for the next launch
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(ctrl + 2, 1);
    if (prev == (int)gridDim.x - 1) {
      // every CTA of this launch has read its targets: move them to where the counters stand after this launch
      ctrl[2] = 0;
      for (int t = 0; t < num_tiles; ++t)
        if (p.oneshot || t % p.world == p.rank) targets[t] += p.world * per_tile;     // only counters that received arrivals
      if (!p.oneshot) targets[p.lay.tiles_max] += num_tiles * n_chunks;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Greedy sampling over vocabulary-parallel logits without gathering them: every rank reduces its own logits
// shard to (max, argmax, running max, sum of exponentials) per row, writes the four numbers into every rank's
// buffer, and after a counter barrier every rank combines the `world` candidates (lowest token id wins ties).
// Exchanges 16 bytes per row and rank instead of the reference's all-gather of the full logits
// (server/lorax_server/layers/tensor_parallel.py:50-79).
// ------------------------------------------------------------------------------------------------
struct ArgmaxTpParams {
  unsigned char* peers[kArMaxRanks];
  long long cand_off;     // float4 [world][max_rows]
  long long ctrl_off;     // int [8]: 3 = arrival counter, 5 = cta_done
  long long target_off;   // running target of the arrival counter at index tiles_max + 1
  int tiles_max;
  int rank, world, max_rows;
  const __nv_bfloat16* logits;
  long long ld;
  int T, V_local, vocab_start;
  int* ids;
  float* logprobs;
  int* status;
  unsigned long long budget_ns;        // how long a wait for another GPU lasts before the kernel gives up
};

__global__ void __launch_bounds__(512) argmax_tp_kernel(const ArgmaxTpParams p) {
  const int t = blockIdx.x;
  unsigned char* local = p.peers[p.rank];
  int* ctrl = reinterpret_cast<int*>(local + p.ctrl_off);
  int* target = reinterpret_cast<int*>(local + p.target_off) + p.tiles_max + 1;
  const __nv_bfloat16* row = p.logits + t * p.ld;
  float best = -INFINITY, m = -INFINITY, s = 0.f;
  int besti = 0x7fffffff;
  for (int i = threadIdx.x; i < p.V_local; i += blockDim.x) {
    const float x = __bfloat162float(row[i]);
    if (x > best || (x == best && i < besti)) { best = x; besti = i; }
    if (x > m) { s = s * __expf(m - x) + 1.f; m = x; } else s += __expf(x - m);
  }
  __shared__ float sb[16], sm[16], ss[16];
  __shared__ int si[16];
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o), om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { sb[w] = best; si[w] = besti; sm[w] = m; ss[w] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
      if (sb[i] > best || (sb[i] == best && si[i] < besti)) { best = sb[i]; besti = si[i]; }
      const float nm = fmaxf(m, sm[i]);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (sm[i] == -INFINITY ? 0.f : ss[i] * __expf(sm[i] - nm));
      m = nm;
    }
    const float4 cand = make_float4(best, __int_as_float(besti + p.vocab_start), m, s);
    for (int r = 0; r < p.world; ++r) {
      float4* dst = reinterpret_cast<float4*>(p.peers[r] + p.cand_off) + (long long)p.rank * p.max_rows + t;
      *dst = cand;
    }
    __threadfence_system();
    for (int r = 0; r < p.world; ++r) red_release_sys_add(reinterpret_cast<int*>(p.peers[r] + p.ctrl_off) + 3, 1);
    // all rows of all ranks: world * T arrivals per launch
    if (wait_counter(ctrl + 3, *target + p.world * p.T, p.status, 3000 + t, p.budget_ns)) {
      const float4* c = reinterpret_cast<const float4*>(local + p.cand_off);
      float gb = -INFINITY, gm = -INFINITY, gs = 0.f;
      int gi = 0x7fffffff;
      for (int r = 0; r < p.world; ++r) {
        const float4 v = __ldcg(c + (long long)r * p.max_rows + t);
        const int idx = __float_as_int(v.y);
        if (v.x > gb || (v.x == gb && idx < gi)) { gb = v.x; gi = idx; }
        const float nm = fmaxf(gm, v.z);
        gs = (gm == -INFINITY ? 0.f : gs * __expf(gm - nm)) + (v.z == -INFINITY ? 0.f : v.w * __expf(v.z - nm));
        gm = nm;
      }
      p.ids[t] = gi;
      if (p.logprobs) p.logprobs[t] = gb - (gm + __logf(gs));
    }
    __threadfence();
    const int prev = atomicAdd(ctrl + 5, 1);
    if (prev == (int)gridDim.x - 1) { ctrl[5] = 0; *target += p.world * p.T; __threadfence(); }
  }
}

typedef CUresult (*EncodeTiledFn3)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn3 encode_fn3() {
  static EncodeTiledFn3 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn3>(ptr);
  }
  return fn;
}
static int make_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn3 fn = encode_fn3();
  if (!fn) return -1;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kArBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}

template <int BN, int STAGES>
static int launch_ar(const CUtensorMap& tw, const CUtensorMap& tx, const ArParams& p, int num_sms, cudaStream_t s) {
  using S = ArSmem<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_allreduce_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    configured = true;
  }
  const int num_tiles = (p.N + kArBM - 1) / kArBM;
  const int tok_chunk = p.oneshot ? kArTokChunkOne : kArTokChunkTwo;
  const int n_chunks = (p.T + tok_chunk - 1) / tok_chunk;
  const int n_owned = p.oneshot ? num_tiles : (num_tiles + p.world - 1) / p.world;
  const int units = num_tiles * p.ttiles * p.ksplit;
  int grid = units > n_owned * n_chunks ? units : n_owned * n_chunks;
  if (grid > num_sms) grid = num_sms;          // all CTAs must be co-resident: they wait on peers
  gemm_allreduce_kernel<BN, STAGES><<<grid, kArThreads, S::kTotal, s>>>(tw, tx, p);
  return -(int)cudaGetLastError();
}

}  // namespace lx

extern "C" {

int lx_ar_max_tokens() { return lx::kArMaxTokens; }

// Bytes of symmetric memory a rank must provide for outputs up to n_max features, and the offsets inside it
// (written to layout_out[0..7]: recv_off, out_off, arrived_off, ctrl_off, tiles_owned_max, cand_off, target_off, tiles_max).
long long lx_ar_layout(int world, int n_max, int max_rows, long long* layout_out) {
  using namespace lx;
  const int tiles_max = (n_max + kArBM - 1) / kArBM;
  const int tiles_owned_max = (tiles_max + world - 1) / world;
  long long off = 0;
  {
    const long long two_shot = (long long)kArMaxSlots * tiles_owned_max * kArMaxTokens * kArBM * 4;
    const long long one_shot = (long long)kArMaxSlots * tiles_max * kArOneShotTokens * kArBM * 4;
    layout_out[0] = off; off += two_shot > one_shot ? two_shot : one_shot;
  }
  layout_out[1] = off; off += (long long)kArMaxTokens * n_max * 2;
  off = (off + 255) & ~255ll;
  layout_out[2] = off; off += (long long)tiles_max * 4;
  off = (off + 255) & ~255ll;
  layout_out[3] = off; off += 64;
  layout_out[4] = tiles_owned_max;
  off = (off + 255) & ~255ll;
  layout_out[5] = off; off += (long long)world * max_rows * 16;
  off = (off + 255) & ~255ll;
  layout_out[6] = off; off += (long long)(tiles_max + 2) * 4;
  layout_out[7] = tiles_max;
  return (off + 255) & ~255ll;
}

// out (in the symmetric buffer of every rank, [T, n_max] bf16 at layout.out_off) = all-reduce over ranks of
// x[T, K] @ w[N, K]^T (+ addend) (+ bias).  T <= 256.  Must be launched by every rank of the group, in the same order.
int lx_gemm_allreduce(const void* x, long long ldx, const void* w, long long ldw, const void* bias, const void* addend, long long lda,
                      int T, int N, int K, const unsigned long long* peer_ptrs, int rank, int world, const long long* layout, int n_max,
                      int* status, int num_sms, void* stream) {
  using namespace lx;
  if (T <= 0 || N <= 0) return 0;
  if (T > kArMaxTokens || world > kArMaxRanks || N > n_max) return -1;
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return -2;
  ArParams p{};
  for (int r = 0; r < world; ++r) p.peers[r] = reinterpret_cast<unsigned char*>(peer_ptrs[r]);
  p.lay.recv_off = layout[0]; p.lay.out_off = layout[1]; p.lay.arrived_off = layout[2]; p.lay.ctrl_off = layout[3];
  p.lay.tiles_owned_max = (int)layout[4]; p.lay.n_max = n_max;
  p.lay.target_off = layout[6]; p.lay.tiles_max = (int)layout[7];
  p.rank = rank; p.world = world; p.T = T; p.N = N; p.K = K;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.addend = reinterpret_cast<const __nv_bfloat16*>(addend);
  p.lda = lda;
  p.status = status;
  p.budget_ns = host_wait_budget_ns();
  // token tile: the whole batch when it is small, otherwise 64-token tiles so that phase A spreads over the machine
  // (N / 128 feature tiles alone would occupy a quarter of the SMs)
  const int bn = T <= 16 ? 16 : T <= 32 ? 32 : 64;
  p.ttiles = (T + bn - 1) / bn;
  p.umma_n = T >= bn ? bn : (T + 15) / 16 * 16;
  p.oneshot = T <= kArOneShotTokens ? 1 : 0;
  p.tok_cap = p.oneshot ? kArOneShotTokens : kArMaxTokens;
  p.tiles_cap = p.oneshot ? p.lay.tiles_max : p.lay.tiles_owned_max;
  // K splits: their partial sums travel to the owner exactly like the other ranks' partials, so splitting K costs no
  // extra pass; use it to spread short batches over the machine
  {
    const int tiles = (N + kArBM - 1) / kArBM, kblocks = (K + kArBK - 1) / kArBK;
    int ks = 1;
    while (tiles * p.ttiles * ks * 2 <= num_sms && kblocks / (ks * 2) >= 4 && world * ks * 2 <= kArMaxSlots) ks *= 2;
    p.ksplit = ks;
  }
  CUtensorMap tw, tx;
  if (make_map(&tw, w, N, K, ldw, kArBM)) return -3;
  if (make_map(&tx, x, T, K, ldx, bn)) return -4;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (bn) {
    case 16: return launch_ar<16, 8>(tw, tx, p, num_sms, s);
    case 32: return launch_ar<32, 8>(tw, tx, p, num_sms, s);
    default: return launch_ar<64, 8>(tw, tx, p, num_sms, s);
  }
}

// ids[T], logprobs[T] = greedy choice over the full vocabulary from vocabulary-parallel logits [T, V_local].
int lx_argmax_tp(const void* logits, long long ld, int T, int V_local, int vocab_start, int* ids, float* logprobs,
                 const unsigned long long* peer_ptrs, int rank, int world, const long long* layout, int max_rows, int* status, void* stream) {
  using namespace lx;
  if (T <= 0) return 0;
  if (T > max_rows || world > kArMaxRanks) return -1;
  ArgmaxTpParams p{};
  for (int r = 0; r < world; ++r) p.peers[r] = reinterpret_cast<unsigned char*>(peer_ptrs[r]);
  p.cand_off = layout[5]; p.ctrl_off = layout[3]; p.target_off = layout[6]; p.tiles_max = (int)layout[7];
  p.rank = rank; p.world = world; p.max_rows = max_rows;
  p.logits = reinterpret_cast<const __nv_bfloat16*>(logits); p.ld = ld; p.T = T; p.V_local = V_local; p.vocab_start = vocab_start;
  p.ids = ids; p.logprobs = logprobs; p.status = status;
  p.budget_ns = host_wait_budget_ns();
  argmax_tp_kernel<<<T, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);     // T <= 512 rows: all CTAs co-resident
  return -(int)cudaGetLastError();
}

}  // extern "C"
