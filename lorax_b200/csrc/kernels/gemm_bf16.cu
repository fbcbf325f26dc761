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
// Multi-adapter LoRA rides in the same launch (template flag LORA, weights on the M side).  The reference runs a shrink kernel,
// the base GEMM and an expand kernel per projection and rank group (server/lorax_server/utils/layers.py:114-164).  Here
//   * the shrink, v = x A_cat^T for the few rows of a decode-sized step, is computed by the four epilogue warps while the first
//     K loop runs (they would wait for the accumulator otherwise): matrix-vector work on mma.sync with operands loaded
//     straight from global memory, written as bf16 images already in the shared-memory layout of a UMMA operand;
//   * the expand is added after the K loop of every base tile by further UMMAs (B_cat tile of the adapter x that image,
//     K = rank) straight into the TMEM accumulator, so the epilogue is unchanged and the output is written once.
// The operands of those UMMAs are 32-byte-swizzled K slices of 16 ranks (4 KB of B_cat, 1.5 KB of image), up to eight per
// pipeline stage.  B_cat tiles of every adapter come through four arena-wide tensor maps (one per rank class) that are kernel
// parameters: a third coordinate, in 16-byte steps, says where the adapter's B_cat starts, so no per-adapter descriptor is
// fetched or fenced.  The list of a token tile's units is built once per CTA and reused for every feature tile.  A CTA counts
// itself in when its shrink units are done and the first expand stage of a CTA waits until every CTA of the launch has; the
// launch has at most one CTA per SM, all resident, and the shrink waits for nothing, so that wait cannot deadlock, and it is
// bounded like the others.  When that wait cannot be used (no counters, blobs the arena-wide maps cannot address) a launch of
// `lora_shrink_rows_kernel` in front of the GEMM writes the images instead.
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

struct LoraTileG { int slot, row0, nrows, pad; };

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
  // Multi-adapter LoRA in the same launch (LORA kernels only; lora_tiles == nullptr otherwise).  Rows of the step are grouped
  // by adapter: the table holds (slot, first row, rows <= 32, -) entries, live ones first, then entries with slot < 0.
  const LoraTileG* lora_tiles;
  int lora_num_tiles;
  const CUtensorMap* lora_slot_tmaps;  // [num_slots][maps_per_slot]: {K, nparts * r, layers} of A_cat and {r, N, layers} of B_cat
  int lora_maps_per_slot, lora_map_a, lora_map_b;
  const int* lora_slot_rank;
  const long long* lora_slot_base;
  int lora_num_slots;
  int lora_nparts, lora_n0, lora_n1;   // parts of the fused projection (q | k | v, gate | up) and their boundaries (multiples of 128)
  int lora_layer;
  __nv_bfloat16* lora_vimg;            // [part][4 K slices][entry][48 rows][16] bf16: v as K-major, 32-byte-swizzled UMMA operand images
  long long lora_off_b;                // B_cat of the group and layer: slot_base + rank * lora_off_b (elements)
  long long lora_off_a;                // A_cat likewise
  const __nv_bfloat16* lora_arena;     // the slots' blobs
  const __nv_bfloat16* lora_x;         // the step's activations [T, K] (operand B of the GEMM), row stride lora_ldx
  long long lora_ldx;
  int lora_max_r;                      // largest rank * parts of a resident adapter: bounds the 8-row blocks of a shrink unit
  int lora_inline_shrink;              // 1: the epilogue warps compute the shrink during the first K loop (0: a launch in front did)
  int* lora_sync;                      // [2] CTAs of this launch that have finished / whose shrink units are done; zero between launches
  int lora_arena_maps;                 // 1: B_cat tiles come through the four arena-wide maps of the launch (LoraBMaps), not the slots' own
  int lora_fence_maps;                 // 1: acquire-fence a slot's B_cat map before every use (0: never; measurement only)
  int lora_skip;                       // measurement only: bit 0 leaves out the shrink launch, bit 1 the expand stages (results are then wrong)
  int lora_T;                          // rows of the step
};

// ---- LoRA items ----------------------------------------------------------------------------------------------
constexpr int kLoraWin = 48;            // a run of <= 32 rows lies inside a 16-aligned window of at most 48 rows
constexpr int kLoraSliceElems = kLoraWin * 16;      // one K slice (16 ranks) of an image: 48 rows of 32 bytes
constexpr int kLoraSliceBytes = kLoraSliceElems * 2;
constexpr int kLoraImgElems = 4 * kLoraSliceElems;  // ranks up to 64
constexpr int kLoraBTileBytes = kBM * 32;           // 128 features x 16 ranks of B_cat
constexpr int kLoraUnitBytes = kLoraBTileBytes + kLoraSliceBytes;     // what one expand unit occupies in a pipeline stage

LX_DEVICE int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
LX_DEVICE void st_release_gpu(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
LX_DEVICE void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

LX_DEVICE void red_release_gpu_add(int* p, int v) { asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
// K-major operand with 32-byte swizzle: rows of 32 bytes (16 bf16), 8-row groups 256 bytes apart.
LX_DEVICE uint64_t make_desc_k_sw32(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(256 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(6) << 61;
  return d;
}

// The table of the step, checked once per CTA and kept in shared memory: the producer and the MMA thread walk it for every
// base tile, and a walk through global memory (entry -> slot -> rank, each a trip to L2) costs more than the tile itself.
constexpr int kLoraMaxEntries = 512;
struct LoraEnt { int slot, row0; short nrows, r; int boff; };    // r == 0: nothing to do for the entry; slot < 0: end of the live entries
static_assert(sizeof(LoraEnt) == 16, "one 16-byte word per entry");
LX_DEVICE void load_lora_entries(const GemmParams& p, LoraEnt* ents, int* n_live) {
  for (int lt = threadIdx.x; lt < p.lora_num_tiles; lt += blockDim.x) {
    const LoraTileG t = p.lora_tiles[lt];
    if (t.slot < 0) atomicMin(n_live, lt);
    LoraEnt e{t.slot, t.row0, (short)max(min(min(t.nrows, 32), p.lora_T - t.row0), -1), 0, 0};
    if (t.slot >= 0 && t.slot < p.lora_num_slots && e.nrows > 0 && t.row0 >= 0) {
      const int r = p.lora_slot_rank[t.slot];
      const long long base = p.lora_slot_base[t.slot];
      if (r > 0 && r <= 64 && (r & 15) == 0 && base >= 0) {
        const long long b = base + (long long)r * p.lora_off_b;      // first element of B_cat, as a coordinate in 16-byte steps
        if (p.lora_arena_maps && ((b & 7) != 0 || (b >> 3) > 0x7fffffffll)) {
          report_status(p.status, kBadIndex, lt);                    // a blob that the arena-wide maps cannot address
        } else {
          e.r = (short)r;
          e.boff = (int)(b >> 3);
        }
      }
    }
    ents[lt] = e;
  }
}

// The part of table entry `lt` that adds to accumulator columns [c0, c1) of the token tile whose rows are [j0, jlim).
struct ExpandItem {
  int slot, r, w0, c0, c1, boff;
};
// -1: end of the live entries or of those that can meet the tile (they are sorted by row), 0: nothing to add for this
// entry, 1: `e` is valid.
LX_DEVICE int decode_expand_item(const LoraEnt* ents, int lt, int j0, int jlim, ExpandItem& e) {
  const LoraEnt t = ents[lt];
  if (t.slot < 0 || t.row0 >= jlim) return -1;
  if (t.r == 0) return 0;
  e.slot = t.slot;
  e.r = t.r;
  e.boff = t.boff;
  e.w0 = t.row0 & ~15;
  const int w1 = (t.row0 + t.nrows + 15) & ~15;
  e.c0 = max(e.w0, j0);
  e.c1 = min(w1, jlim);
  if (e.c0 >= e.c1) return 0;
  return 1;
}

// One unit of work of a CTA: k-blocks [kb0, kb1) of one output tile.  nparts == 0: the CTA owns the whole tile and
// writes bf16 directly.  Otherwise the fp32 partial goes to `part_off` (floats from ws), the arrival is counted in
// counters[counter], and the last of the nparts contributors sums partials red_base + i * red_stride
// (i = 0 .. nparts-1; the first one at red_first instead) in that fixed order.
struct GemmWork {
  int tile, kb0, kb1, nparts, counter, part_idx;     // part_idx: which of the nparts contributors this CTA is
  long long part_off, red_first, red_base, red_stride;
};

// A stream-K tile the CTA has parked a partial for: summed after the CTA's last unit of work.
struct PendingTile {
  int ta, tb, counter, nparts, part_idx;
  long long red_first, red_base, red_stride;
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
      w.part_idx = split;
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
    w.part_idx = cta - first;
    w.counter = r;
    w.part_off = (long long)(cta * 2 + (first_seg ? 0 : 1)) * kPart;
    w.red_base = (long long)(first * 2) * kPart;
    w.red_stride = 2 * kPart;
    w.red_first = w.red_base + (sk_start(first) < t0 ? kPart : 0);
    return true;
  }
};

// ---- shrink units, computed by the epilogue warps while the first K loop runs -----------------------------------------------
// v = A_cat(slot) x for the rows of the step: the rows are few, the work is bound by how fast A_cat streams in, and the four
// epilogue warps have nothing to do until the first accumulator is complete.  A unit is (a group of up to eight rows of one
// table entry, 16 rank rows): the four warps split K in 32-element blocks, a lane loads 16 bytes of two rank rows and of one
// row of x straight from global memory (no staging, no barrier inside the K loop) and feeds them to two mma.sync m16n8k16
// (the order of k inside a block is permuted the same way for both operands, which a dot product does not see); the loads of
// the next eight blocks are in flight while the current eight are multiplied.  The warps' partial sums meet in shared memory
// and go straight into the operand images the expand stages read.  Units are dealt round-robin over the CTAs of the launch;
// a CTA counts itself in when its units are done (see lora_sync).
constexpr int kShrinkRows = 8;          // rows of x per mma (its N); a unit has one such group, or four of them in long steps
// Rows of x per shrink unit.  Decode-sized steps have few rows per adapter: one group of eight.  Long steps (prefill) have whole
// entries of 32 rows: four groups share every load of the A_cat block, which halves the bytes a unit of work moves.
LX_DEVICE int lora_shrink_unit_rows(const GemmParams& p) { return p.lora_T > 512 ? 4 * kShrinkRows : kShrinkRows; }
LX_DEVICE void lora_group_prefix(const GemmParams& p, const LoraEnt* ents, unsigned short* gstart) {
  const int unit_rows = lora_shrink_unit_rows(p);
  const int lane = threadIdx.x & 31;
  int run = 0;
  for (int lt0 = 0; lt0 < p.lora_num_tiles; lt0 += 32) {
    const int lt = lt0 + lane;
    int cnt = 0;
    if (lt < p.lora_num_tiles) {
      const LoraEnt e = ents[lt];
      if (e.slot >= 0 && e.r > 0) cnt = (e.nrows + unit_rows - 1) / unit_rows;
    }
    int incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    if (lt < p.lora_num_tiles) gstart[lt] = (unsigned short)(run + incl - cnt);
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) gstart[p.lora_num_tiles] = (unsigned short)run;
}

struct ShrinkUnit {
  int lt, t0, nt, r, j;          // entry, first row, rows (<= 8 or 32), rank of the slot, first of the unit's 16 rank rows (part * r + i)
  const __nv_bfloat16* a;        // A_cat row j
};

LX_DEVICE bool decode_shrink_unit(const GemmParams& p, const LoraEnt* ents, const unsigned short* gstart, int u, int nblk, int unit_rows,
                                  ShrinkUnit& s) {
  const int g = u / nblk, jb = u - g * nblk;
  int lo = 0, hi = p.lora_num_tiles;                     // last entry with gstart <= g
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if ((int)gstart[mid] <= g) lo = mid; else hi = mid;
  }
  const LoraEnt e = ents[lo];
  if (e.slot < 0 || e.r <= 0) return false;
  const int sub = g - (int)gstart[lo];
  if (sub * unit_rows >= e.nrows || jb * 16 >= e.r * p.lora_nparts) return false;
  s.lt = lo;
  s.t0 = e.row0 + sub * unit_rows;
  s.nt = min(unit_rows, e.row0 + e.nrows - s.t0);
  s.r = e.r;
  s.j = jb * 16;
  s.a = p.lora_arena + (long long)e.boff * 8 + (long long)e.r * (p.lora_off_a - p.lora_off_b) + (long long)s.j * p.K;
  return true;
}

LX_DEVICE void mma_bf16_16x8x16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The loads of SB K blocks of this warp (blocks ewarp + 4 * (SB * batch + i)): rank rows g and g + 8 of A_cat, row g of each of
// the unit's NG groups of x.  NG * SB stays 8 or 16 so that the loads in flight fill the same registers either way.
template <int NG, int SB>
LX_DEVICE void shrink_loads(const GemmParams& p, const ShrinkUnit& s, int batch, int ewarp, int lane, uint4* ra, uint4* rb, uint4 (*rx)[SB]) {
  const int K8 = p.K >> 3;
  const int g = lane >> 2, t = lane & 3;
  const uint4* a0 = reinterpret_cast<const uint4*>(s.a + (long long)g * p.K);
  const uint4* a1 = reinterpret_cast<const uint4*>(s.a + (long long)(g + 8) * p.K);
#pragma unroll
  for (int i = 0; i < SB; ++i) {
    const int kk = (ewarp + 4 * (SB * batch + i)) * 4 + t;          // 16-byte index inside the row
    const bool in = kk < K8;
    ra[i] = in ? __ldg(a0 + kk) : make_uint4(0, 0, 0, 0);
    rb[i] = in ? __ldg(a1 + kk) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int q = 0; q < NG; ++q) {
      const int row = q * kShrinkRows + g;
      const uint4* xr = reinterpret_cast<const uint4*>(p.lora_x + (long long)(s.t0 + row) * p.lora_ldx);
      rx[q][i] = (in && row < s.nt) ? xr[kk] : make_uint4(0, 0, 0, 0);
    }
  }
}

template <int NG, int SB>
LX_DEVICE void lora_shrink_units_t(const GemmParams& p, const LoraEnt* ents, const unsigned short* gstart, float* red, int ewarp, int lane) {
  const int tid4 = ewarp * 32 + lane;
  const int nblk = (p.lora_max_r + 15) >> 4;
  const int U = (int)gstart[p.lora_num_tiles] * nblk;
  const int nbatch = ((p.K + 31) / 32 + 4 * SB - 1) / (4 * SB);    // batches of SB blocks per warp
  constexpr int kUnitRows = NG * kShrinkRows;
  ShrinkUnit cur;
  int u = (int)blockIdx.x;
  while (u < U && !decode_shrink_unit(p, ents, gstart, u, nblk, kUnitRows, cur)) u += (int)gridDim.x;
  if (u < U) {
    int b = 0, par = 0;
    uint4 ra[SB], rb[SB], rx[NG][SB];
    shrink_loads<NG, SB>(p, cur, 0, ewarp, lane, ra, rb, rx);
    float acc[NG][4];
#pragma unroll
    for (int q = 0; q < NG; ++q) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
    while (true) {
      // the batch after this one: the next of the unit, or the first of the CTA's next unit
      ShrinkUnit nxt = cur;
      int nb = b + 1, nu = u;
      bool more = true;
      if (nb == nbatch) {
        nb = 0;
        nu = u + (int)gridDim.x;
        while (nu < U && !decode_shrink_unit(p, ents, gstart, nu, nblk, kUnitRows, nxt)) nu += (int)gridDim.x;
        more = nu < U;
      }
      uint4 na[SB], nbv[SB], nx[NG][SB];
      if (more) shrink_loads<NG, SB>(p, nxt, nb, ewarp, lane, na, nbv, nx);
#pragma unroll
      for (int i = 0; i < SB; ++i) {
#pragma unroll
        for (int q = 0; q < NG; ++q) {
          if (q * kShrinkRows < cur.nt) {
            mma_bf16_16x8x16(acc[q], ra[i].x, rb[i].x, ra[i].y, rb[i].y, rx[q][i].x, rx[q][i].y);
            mma_bf16_16x8x16(acc[q], ra[i].z, rb[i].z, ra[i].w, rb[i].w, rx[q][i].z, rx[q][i].w);
          }
        }
      }
      if (b == nbatch - 1) {
        // the unit is complete: 16 ranks x up to 8 rows per group.  This warp holds (rank g, rows 2t, 2t+1) and (rank g + 8, same
        // rows) of every group; the groups go through the two staging buffers one after the other.
        const LoraEnt e = ents[cur.lt];
        const int w0 = e.row0 & ~15;
        const int wn = ((e.row0 + e.nrows + 15) & ~15) - w0;
        const int pp = cur.j / cur.r, i0 = cur.j - pp * cur.r;
        __nv_bfloat16* img = p.lora_vimg + ((long long)(pp * 4 + (i0 >> 4)) * p.lora_num_tiles + cur.lt) * kLoraSliceElems;
#pragma unroll
        for (int q = 0; q < NG; ++q) {
          if (q * kShrinkRows < cur.nt) {              // the same for the four warps: they meet at the barrier below
            const int t0g = cur.t0 + q * kShrinkRows;
            const int ntg = min(kShrinkRows, cur.nt - q * kShrinkRows);
            const int g = lane >> 2, t = lane & 3;
            float* mine = red + (par * 4 + ewarp) * 128;                // [16 ranks][8 rows]
            mine[g * 8 + 2 * t] = acc[q][0];
            mine[g * 8 + 2 * t + 1] = acc[q][1];
            mine[(g + 8) * 8 + 2 * t] = acc[q][2];
            mine[(g + 8) * 8 + 2 * t + 1] = acc[q][3];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid4 < 2 * ntg) {
              // thread -> (row rq of the group, 8 ranks ch): one 16-byte chunk of the image
              const int rq = tid4 >> 1, ch = tid4 & 1;
              const float* r0 = red + par * 4 * 128;
              float v[8];
#pragma unroll
              for (int h = 0; h < 8; ++h) {
                const int o = (ch * 8 + h) * 8 + rq;
                v[h] = r0[o] + r0[128 + o] + r0[256 + o] + r0[384 + o];
              }
              const int cr = t0g + rq - w0;
              *reinterpret_cast<uint4*>(img + cr * 16 + ((ch ^ ((cr >> 2) & 1)) << 3)) =
                  make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
            }
            // rows of the window outside the entry: [0, z_lo) with the entry's first group, [z_hi, wn) with its last
            const int z_lo = (t0g == e.row0) ? e.row0 - w0 : 0;
            const int z_hi = (t0g + ntg == e.row0 + e.nrows) ? e.row0 + e.nrows - w0 : wn;
            const int zrows = z_lo + (wn - z_hi);
            if (tid4 >= 32 && tid4 - 32 < 2 * zrows) {
              const int cz = (tid4 - 32) >> 1, ch = (tid4 - 32) & 1;
              const int row = cz < z_lo ? cz : z_hi + (cz - z_lo);
              *reinterpret_cast<uint4*>(img + row * 16 + (ch << 3)) = make_uint4(0, 0, 0, 0);
            }
            par ^= 1;
            acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
          }
        }
      }
      if (!more) break;
      cur = nxt; b = nb; u = nu;
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        ra[i] = na[i]; rb[i] = nbv[i];
#pragma unroll
        for (int q = 0; q < NG; ++q) rx[q][i] = nx[q][i];
      }
    }
  }
  // this CTA's units are done: make the images visible to the bulk copies of every CTA, then count in
  __threadfence();
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (tid4 == 0) {
    fence_proxy_async_all();
    red_release_gpu_add(&p.lora_sync[1], 1);
  }
}

LX_DEVICE void lora_shrink_units(const GemmParams& p, const LoraEnt* ents, const unsigned short* gstart, float* red, int ewarp, int lane) {
  if (lora_shrink_unit_rows(p) == kShrinkRows) lora_shrink_units_t<1, 8>(p, ents, gstart, red, ewarp, lane);
  else lora_shrink_units_t<4, 4>(p, ents, gstart, red, ewarp, lane);
}

// Bounded wait for *flag == want.  False when the budget ran out.
LX_DEVICE bool wait_flag(const int* flag, int want, volatile int* abort_flag) {
  uint64_t t0 = 0;
  uint32_t polls = 0;
  while (ld_acquire_gpu(flag) != want) {
    if ((++polls & 255u) == 0) {
      if (abort_flag != nullptr && *abort_flag != 0) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitBudgetNs) return false;
    }
  }
  return true;
}

// ---- expand units, built by a whole warp ------------------------------------------------------------------------
// A unit = one K slice (16 ranks) of one table entry that meets the token tile.  The producer warp and the MMA warp each build
// the same list in their own shared-memory area, 32 entries at a time (one per lane, ranks -> slices by a warp prefix sum), and
// keep it while the token tile stays the same: it does not depend on the feature tile.
// First live entry whose 16-aligned window ends after row j0 (entries are sorted by row and do not overlap).
LX_DEVICE int lora_first_entry(const LoraEnt* ents, int n_live, int j0) {
  int lo = 0, hi = n_live;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    const LoraEnt t = ents[mid];
    if (((t.row0 + t.nrows + 15) & ~15) > j0) hi = mid; else lo = mid + 1;
  }
  return lo;
}

struct LoraUnit {
  int slot, img;        // img = entry * 4 + slice
  int c0, c1;           // accumulator columns [c0, c1) the unit adds to
  int w0;               // first row of the entry's 16-aligned window
  int boff;             // B_cat of the slot, group and layer in 16-byte steps from the arena's start
  int rclass;           // rank / 16 - 1: which arena-wide map has the slot's row pitch
  int pad_;
};
static_assert(sizeof(LoraUnit) == 32, "two 16-byte words per unit");
// The units of one expand stage travel in the stage itself, behind its tiles: the producer warp builds the list, the MMA thread
// reads what to issue after the stage's barrier.  `last` closes the run of expand stages of a tile.
struct LoraStageHeader {
  LoraUnit units[8];
  int nu, last, pad_[2];
};
constexpr int kLoraListCap = 256;       // units a list holds; it is worked off whenever it holds 128 or more
LX_DEVICE int lora_build_units(const GemmParams& p, const LoraEnt* ents, int lt0, int j0, int jlim, LoraUnit* list, int n, bool& ended) {
  const int lane = threadIdx.x & 31;
  const int lt = lt0 + lane;
  ExpandItem e;
  const int rc = lt < p.lora_num_tiles ? decode_expand_item(ents, lt, j0, jlim, e) : -1;
  const unsigned endmask = __ballot_sync(0xffffffffu, rc < 0);
  const int first_end = endmask ? __ffs(endmask) - 1 : 32;
  const int nsl = (rc == 1 && lane < first_end) ? e.r / 16 : 0;
  int incl = nsl;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  const int excl = incl - nsl;
  const int total = __shfl_sync(0xffffffffu, incl, 31);
  for (int sl = 0; sl < nsl; ++sl) {
    const int idx = n + excl + sl;
    if (idx < kLoraListCap) list[idx] = LoraUnit{e.slot, lt * 4 + sl, e.c0, e.c1, e.w0, e.boff, e.r / 16 - 1, 0};
  }
  ended = endmask != 0;
  __syncwarp();
  return min(n + total, kLoraListCap);
}

// The complete unit list of token tile [j0, jlim), if it fits the list: built ahead of time (before the kernel waits for its
// predecessor) for the CTA's first tile.  Returns the number of units, or -1 when the list would not hold them all.
LX_DEVICE int lora_prebuild_units(const GemmParams& p, const LoraEnt* ents, int n_live, int j0, int jlim, LoraUnit* list) {
  int n = 0;
  bool ended = false;
  for (int lt0 = lora_first_entry(ents, n_live, j0); !ended && lt0 < p.lora_num_tiles; lt0 += 32) {
    if (n > kLoraListCap - 128) return -1;             // 32 entries yield up to 128 units
    n = lora_build_units(p, ents, lt0, j0, jlim, list, n, ended);
  }
  return n;
}

// Pulls the B_cat rows that feature tile `ta` needs for the units of `list` into L2 (whole warp; adapter weights, which no kernel
// of a step writes, so this may run before the kernel in front has drained).
LX_DEVICE void lora_prefetch_b(const GemmParams& p, const LoraUnit* list, int n, int ta) {
  const int rows = min(kBM, p.a_rows - ta * kBM);
  for (int u = threadIdx.x & 31; u < n; u += 32) {
    const LoraUnit q = list[u];
    if ((q.img & 3) == 0) {
      const int r = (q.rclass + 1) * 16;
      const char* src = reinterpret_cast<const char*>(p.lora_arena) + (long long)q.boff * 16 + (long long)ta * kBM * r * 2;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((uint32_t)(rows * r * 2)) : "memory");
    }
  }
}

// B_cat of every slot through one map per rank class: dims {rank, N, arena / 16 bytes} with strides {2 * rank, 16} bytes, box
// {16, 128, 1}, 32-byte swizzle.  The third coordinate is where the slot's B_cat starts, so one descriptor, passed as a kernel
// parameter, serves every adapter: nothing to fetch from memory per slot and nothing to fence.
struct LoraBMaps { CUtensorMap m[4]; };

LX_DEVICE void tensormap_fence_acquire_g(const CUtensorMap* m) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

template <int BN, int STAGES, bool LORA>
struct GemmSmem {
  static constexpr int kBRows = (LORA && BN < 64) ? 64 : BN;      // a LoRA stage holds a 48-row image in the B region
  static constexpr int kAcc = kBRows;                             // TMEM columns per accumulator (a shrink item needs 48)
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // expand units that share a stage: B_cat tiles first, then the image slices
  static constexpr int kUnits = (kStageBytes / kLoraUnitBytes) < 8 ? (kStageBytes / kLoraUnitBytes) : 8;
  static constexpr int kBarrierBytes = 256;
  // entry table, two unit lists, groups-before-entry prefix (shrink units)
  static constexpr int kShrinkBytes = LORA ? (kLoraMaxEntries + 8) * 2 : 0;
  static constexpr int kEntBytes = LORA ? kLoraMaxEntries * (int)sizeof(LoraEnt) + kLoraListCap * 32 + kShrinkBytes : 0;
  static_assert(!LORA || kStageBytes - kUnits * kLoraUnitBytes >= (int)sizeof(LoraStageHeader), "room for the unit list behind the tiles of a stage");
  static constexpr int kEpiBytes = 4 * 32 * 32 * 2;     // per epilogue warp, 32 tokens x 32 features: the transposing store of the weights-on-M path
  static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + kEntBytes + kEpiBytes + 1024;  // +1024 for manual alignment
};

template <int BN, int STAGES, bool LORA>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ LoraBMaps bmaps, const GemmParams p) {
  pdl_trigger();
  using S = GemmSmem<BN, STAGES, LORA>;
  static_assert(S::kTotal <= 227 * 1024, "shared memory of one CTA");
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
  int* n_live = reinterpret_cast<int*>(tmem_base_slot + 3);             // live entries of the LoRA table
  LoraEnt* ents = reinterpret_cast<LoraEnt*>(smem + STAGES * S::kStageBytes + S::kBarrierBytes);
  LoraUnit* ulist_p = reinterpret_cast<LoraUnit*>(ents + kLoraMaxEntries);      // producer warp's expand units of the current token tile
  unsigned short* gstart = reinterpret_cast<unsigned short*>(ulist_p + kLoraListCap);   // [entries + 1] four-row groups before an entry
  __nv_bfloat16* epi_stage = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * S::kStageBytes + S::kBarrierBytes + S::kEntBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = (2 * S::kAcc < 32) ? 32 : 2 * S::kAcc;

  const int tiles_a = (p.a_rows + kBM - 1) / kBM;
  const int tiles_b = (p.b_rows + p.bn - 1) / p.bn;
  const int num_tiles = tiles_a * tiles_b;
  const int kblocks = (p.K + kBK - 1) / kBK;
  const bool lora = LORA && p.lora_tiles != nullptr;
  int pre_tb = -1, pre_n = 0;             // token tile whose unit list the producer warp has built ahead of its first tile

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
    *n_live = LORA ? p.lora_num_tiles : 0;
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
  if constexpr (LORA) {
    // the table, the slot ranks and the slot offsets are written by copies that the stream orders before every kernel, never by
    // the kernel in front of this one: reading them does not have to wait for that kernel to drain
    if (lora) {
      load_lora_entries(p, ents, n_live);
      __syncthreads();
      if (p.lora_inline_shrink && warp == 2) lora_group_prefix(p, ents, gstart);
      if (warp == 0 && !(p.lora_skip & 2)) {
        // the producer warp builds the unit list of its first tile now, under the tail of the kernel in front, and pulls that
        // tile's B_cat rows (adapter weights, which no kernel of the step writes) into L2
        GemmWorkIter<BN> it0(p, num_tiles, kblocks);
        GemmWork w0;
        if (it0.next(w0) && w0.kb0 == 0) {
          const int ta0 = p.b_fastest ? w0.tile / tiles_b : w0.tile % tiles_a;
          const int tb0 = p.b_fastest ? w0.tile % tiles_b : w0.tile / tiles_a;
          const int n0 = lora_prebuild_units(p, ents, *n_live, tb0 * p.bn, tb0 * p.bn + p.umma_n, ulist_p);
          if (n0 >= 0) { pre_tb = tb0; pre_n = n0; }
          if (n0 > 0 && p.lora_arena_maps) lora_prefetch_b(p, ulist_p, n0, ta0);
        }
      }
      __syncthreads();
    }
  }
  pdl_wait();      // barriers, TMEM and descriptors are set up while the previous kernel drains; its data is read from here on

  // Work item w -> (tile, split).  Tiles are ordered with the A tile index fastest inside one B tile so that
  // CTAs running at the same time share the B operand through L2.
  if (warp == 0) {
    // Lane 0 feeds the ring with base k-blocks; the LoRA stages of a tile are fed by the whole warp, one lane per unit.
    const uint64_t pol_a = p.hint_a_first ? policy_evict_first() : policy_evict_last();
    const uint64_t pol_b = p.hint_a_first ? policy_evict_last() : policy_evict_first();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int list_tb = pre_tb, list_n = pre_n;  // token tile whose complete unit list sits in ulist_p
    bool first_tile = pre_tb >= 0;         // its B_cat rows were prefetched before the dependent-launch wait
    bool shrink_seen = false;
    GemmWorkIter<BN> it(p, num_tiles, kblocks);
    GemmWork w;
    while (it.next(w)) {
      const int ta = p.b_fastest ? w.tile / tiles_b : w.tile % tiles_a;
      const int tb = p.b_fastest ? w.tile % tiles_b : w.tile / tiles_a;
      if constexpr (LORA) {
        if (lora && w.kb0 == 0 && !(p.lora_skip & 2)) {
          // the whole warp, while the ring still holds the stages of the tile before: this tile's unit list (kept while the token
          // tile stays the same) and its B_cat rows on their way into L2 under the base k-blocks
          if (list_tb != tb) {
            const int n0 = lora_prebuild_units(p, ents, *n_live, tb * p.bn, tb * p.bn + p.umma_n, ulist_p);
            list_tb = n0 >= 0 ? tb : -1;
            list_n = n0 >= 0 ? n0 : 0;
          }
          if (list_tb == tb && list_n > 0 && p.lora_arena_maps && !first_tile) lora_prefetch_b(p, ulist_p, list_n, ta);
          first_tile = false;
        }
      }
      if (lane == 0 && ok) {
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
      if constexpr (LORA) {
        if (lora && w.kb0 == 0 && !(p.lora_skip & 2)) {
          // the LoRA delta of this tile: one unit per K slice of 16 ranks of every table entry whose rows meet the token tile
          __syncwarp();
          stage = __shfl_sync(0xffffffffu, stage, 0);
          phase = __shfl_sync(0xffffffffu, phase, 0);
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          const int i0 = ta * kBM, j0 = tb * p.bn, jlim = j0 + p.umma_n;
          const int part = min(p.lora_nparts - 1, i0 < p.lora_n0 ? 0 : (i0 < p.lora_n1 ? 1 : 2));
          const long long img_part = (long long)part * 4 * p.lora_num_tiles;      // images: [part][slice][entry][48 x 16]
          if (ok && p.lora_inline_shrink && !shrink_seen) {
            // the images are written by the epilogue warps of every CTA of this launch; all CTAs are resident (one per SM)
            if (lane == 0) {
              if (!wait_flag(&p.lora_sync[1], (int)gridDim.x, abort_flag)) {
                report_status(p.status, kTimeoutSplitK, w.tile);
                *abort_flag = 1;
              }
            }
            __syncwarp();
            ok = (*abort_flag == 0);
            fence_proxy_async_all();       // the images were written with ordinary stores; bulk copies read them
            shrink_seen = true;
          }
          constexpr int kU = S::kUnits;
          // One expand stage: up to kU units, one lane each; the units are written behind the stage's tiles for the MMA thread.
          auto send_stage = [&](int base, int nu, bool last) -> bool {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
              if (lane == 0) {
                report_status(p.status, kTimeoutEmptyBarrier, w.tile);
                *abort_flag = 1;
              }
              return false;
            }
            uint8_t* sa = tiles + stage * S::kStageBytes;
            LoraStageHeader* hdr = reinterpret_cast<LoraStageHeader*>(sa + kU * kLoraUnitBytes);
            LoraUnit q{};
            if (lane < nu) {
              q = ulist_p[base + lane];
              hdr->units[lane] = q;
            }
            if (lane == 0) { hdr->nu = nu; hdr->last = last ? 1 : 0; }
            fence_proxy_async_smem();          // the stage's bytes are written by bulk copies at other times
            __syncwarp();
            if (lane == 0) mbar_expect_tx(&full_bar[stage], (uint32_t)(nu * kLoraUnitBytes));
            __syncwarp();
            // image slices of consecutive entries are consecutive in memory: one copy serves the stage
            const int y0 = __shfl_sync(0xffffffffu, q.img, 0);
            const bool in_row = lane >= nu || (q.img == y0 + 4 * lane && (q.img & 3) == 0);
            const bool one_copy = __all_sync(0xffffffffu, in_row);
            if (lane < nu) {
              if (p.lora_arena_maps) {
                tma_load_3d(sa + lane * kLoraBTileBytes, &bmaps.m[q.rclass], &full_bar[stage], (q.img & 3) * 16, i0, q.boff);
              } else {
                const CUtensorMap* mb = p.lora_slot_tmaps + (long long)q.slot * p.lora_maps_per_slot + p.lora_map_b;
                if (p.lora_fence_maps) tensormap_fence_acquire_g(mb);
                tma_load_3d(sa + lane * kLoraBTileBytes, mb, &full_bar[stage], (q.img & 3) * 16, i0, p.lora_layer);
              }
              const long long img = (img_part + (long long)(q.img & 3) * p.lora_num_tiles + (q.img >> 2)) * kLoraSliceElems;
              if (!one_copy) {
                bulk_load_1d(sa + kU * kLoraBTileBytes + lane * kLoraSliceBytes, p.lora_vimg + img, kLoraSliceBytes, &full_bar[stage]);
              } else if (lane == 0) {
                bulk_load_1d(sa + kU * kLoraBTileBytes, p.lora_vimg + img, (uint32_t)(nu * kLoraSliceBytes), &full_bar[stage]);
              }
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            return true;
          };
          // The stages of `n` listed units; the final one is marked when it `closes` the tile (an empty stage if there is no unit).
          auto send_run = [&](int n, bool closes) {
            if (n == 0 && closes) ok = send_stage(0, 0, true);
            for (int base = 0; ok && base < n; base += kU) ok = send_stage(base, min(kU, n - base), closes && base + kU >= n);
          };
          if (!ok) {
          } else if (list_tb == tb) {
            send_run(list_n, true);
          } else {
            // more units than the list holds: built and sent in pieces
            int n = 0;
            bool ended = false;
            for (int lt0 = lora_first_entry(ents, *n_live, j0); ok; lt0 += 32) {
              bool last = true;
              if (lt0 < p.lora_num_tiles) {
                n = lora_build_units(p, ents, lt0, j0, jlim, ulist_p, n, ended);
                last = ended || lt0 + 32 >= p.lora_num_tiles;
                if (n < 128 && !last) continue;
              }
              send_run(n, last);
              if (last) break;
              n = 0;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // Lane 0 issues every MMA.
    const uint32_t idesc = make_idesc(kBM, (uint32_t)p.umma_n, kFmtBF16, kFmtBF16);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    GemmWorkIter<BN> it(p, num_tiles, kblocks);
    GemmWork w;
    while (it.next(w)) {
      const int kb0 = w.kb0, kb1 = w.kb1;
      const uint32_t tmem_d = tmem_base + (uint32_t)(acc * S::kAcc);
      if (lane == 0 && ok) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1, abort_flag)) {
          report_status(p.status, kTimeoutTmemEmpty, w.tile);
          *abort_flag = 1;
          ok = false;
        }
        tc_fence_after();
        for (int kb = kb0; ok && kb < kb1; ++kb) {
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
      }
      if constexpr (LORA) {
        if (lora && kb0 == 0 && !(p.lora_skip & 2) && lane == 0) {
          // the tile's expand stages: each carries its units; the one marked `last` ends the run (there is always one)
          constexpr int kU = S::kUnits;
          const int tb = p.b_fastest ? w.tile % tiles_b : w.tile / tiles_a;
          const int j0 = tb * p.bn;
          bool more = ok;
          while (more) {
            if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
              report_status(p.status, kTimeoutFullBarrier, w.tile);
              *abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
            uint8_t* sp = tiles + stage * S::kStageBytes;
            const LoraStageHeader* hdr = reinterpret_cast<const LoraStageHeader*>(sp + kU * kLoraUnitBytes);
            const uint32_t sa = smem_u32(sp);
            const int nu = min(hdr->nu, kU);
            more = hdr->last == 0;
            for (int u = 0; u < nu; ++u) {
              const LoraUnit q = hdr->units[u];
              const int c0 = q.c0, c1 = q.c1;
              const uint64_t da = make_desc_k_sw32(sa + (uint32_t)(u * kLoraBTileBytes));
              const uint64_t db = make_desc_k_sw32(sa + (uint32_t)(kU * kLoraBTileBytes + u * kLoraSliceBytes + (c0 - q.w0) * 32));
              if (!(p.lora_skip & 32))
                umma_f16_ss(tmem_d + (uint32_t)(c0 - j0), da, db, make_idesc(kBM, (uint32_t)(c1 - c0), kFmtBF16, kFmtBF16), 1u);
            }
            tc_commit(&empty_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
      if (lane == 0 && ok) tc_commit(&tmem_full[acc]);       // accumulator complete
      acc_phase[acc] ^= 1;
      acc ^= 1;
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..5)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool alive = true;
    PendingTile pending[2];
    int n_pending = 0;
    if constexpr (LORA) {
      if (lora && p.lora_inline_shrink) lora_shrink_units(p, ents, gstart, reinterpret_cast<float*>(epi_stage), warp - 2, lane);
    }
    GemmWorkIter<BN> it(p, num_tiles, kblocks);
    GemmWork w;
    while (alive && it.next(w)) {
      const int ta = p.b_fastest ? w.tile / tiles_b : w.tile % tiles_a;
      const int tb = p.b_fastest ? w.tile % tiles_b : w.tile / tiles_a;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc], abort_flag)) {
        report_status(p.status, kTimeoutTmemFull, w.tile);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      acc_phase[acc] ^= 1;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * S::kAcc);
      const int i = ta * kBM + row_in_tile;
      const int j0 = tb * p.bn;
      const int ncols = min(p.bn, p.umma_n);
      const int jend = min(p.b_rows, j0 + ncols);     // columns past it belong to the next tile (or to nobody)
      constexpr int CH = (BN >= 32) ? 32 : 16;
      // Weights on M: a thread holds one feature of CH tokens, the output rows run along the features.  The warp turns its
      // 32 x CH block around in shared memory and stores 16 bytes per lane (8 features of one token) instead of 2.
      const bool turn = p.ldo_a == 1 && (p.ldo_b & 7) == 0 && (p.a_rows & 7) == 0 && (p.bias == nullptr || p.bias_on_a) &&
                        (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;

      if (w.nparts == 0 && turn) {
        __nv_bfloat16* st = epi_stage + quad * (32 * 32);
        const float bias_i = (p.bias != nullptr && i < p.a_rows) ? __bfloat162float(p.bias[i]) : 0.f;
        const int fbase = ta * kBM + quad * 32 + (lane & 3) * 8;
#pragma unroll 1
        for (int c = 0; c < ncols; c += CH) {
          uint32_t r[CH];
          if constexpr (CH == 32) tmem_ld_32x32b_x32(taddr + c, r);
          else tmem_ld_32x32b_x16(taddr + c, r);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < CH; ++q) st[q * 32 + lane] = __float2bfloat16(__uint_as_float(r[q]) * p.out_scale + bias_i);
          __syncwarp();
#pragma unroll
          for (int h = 0; h < CH / 8; ++h) {
            const int tq = h * 8 + (lane >> 2);
            const int t = j0 + c + tq;
            if (t < jend && fbase < p.a_rows) {
              const uint4 val = *reinterpret_cast<const uint4*>(st + tq * 32 + (lane & 3) * 8);
              *reinterpret_cast<uint4*>(p.out + (long long)t * p.ldo_b + fbase) = val;
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      } else if (w.nparts == 0) {
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
        if (p.split_k == 1) {
          // Stream-K: the contributors of a tile are different CTAs that finish at about the same time.  Count in now; after
          // its last unit of work every contributor sums its own share of the tile's columns (see below).
          if (threadIdx.x == 64) atomicAdd(&p.counters[w.counter], 1);
          if (n_pending < 2) pending[n_pending++] = PendingTile{ta, tb, w.counter, w.nparts, w.part_idx, w.red_first, w.red_base, w.red_stride};
          acc ^= 1;
          continue;
        }
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
    // ---- stream-K tiles this CTA contributed to: every contributor sums its share of the columns, 4 rows (16 bytes of
    // every partial) per thread and step.  All contributors are running (one CTA per SM, each a consecutive K range of the
    // same length), so the wait for the others is short; it is bounded like every wait.
    for (int pi = 0; alive && pi < n_pending; ++pi) {
      const PendingTile t = pending[pi];
      if (threadIdx.x == 64) {
        uint64_t t0 = 0;
        uint32_t polls = 0;
        while ((ld_acquire_gpu(&p.counters[t.counter]) & 0xffff) != t.nparts) {
          if ((++polls & 255u) == 0) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitBudgetNs) {
              report_status(p.status, kTimeoutSplitK, t.counter);
              *abort_flag = 1;
              break;
            }
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag != 0) break;
      const int j0 = t.tb * p.bn;
      const int ncols = min(min(p.bn, p.umma_n), p.b_rows - j0);
      const int c_lo = (int)((long long)ncols * t.part_idx / t.nparts), c_hi = (int)((long long)ncols * (t.part_idx + 1) / t.nparts);
      const int tid4 = (int)threadIdx.x - 64;
      const int items = (c_hi - c_lo) * (kBM / 4);
      for (int it0 = tid4; it0 < items; it0 += 128 * 4) {
        // four items per thread and pass, four partials of each in flight
        float4 sum[4];
        long long off[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int it1 = min(it0 + 128 * e, items - 1);
          sum[e] = make_float4(0.f, 0.f, 0.f, 0.f);
          off[e] = (long long)(c_lo + it1 / (kBM / 4)) * kBM + (it1 % (kBM / 4)) * 4;
        }
        for (int sp0 = 0; sp0 < t.nparts; sp0 += 4) {
          float4 v[4][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int sp = min(sp0 + q, t.nparts - 1);
            const float* src = p.ws + (sp == 0 ? t.red_first : t.red_base + sp * t.red_stride);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[q][e] = __ldcg(reinterpret_cast<const float4*>(src + off[e]));
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (sp0 + q < t.nparts) {
#pragma unroll
              for (int e = 0; e < 4; ++e) { sum[e].x += v[q][e].x; sum[e].y += v[q][e].y; sum[e].z += v[q][e].z; sum[e].w += v[q][e].w; }
            }
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int it1 = it0 + 128 * e;
          if (it1 >= items) break;
          const int c = c_lo + it1 / (kBM / 4), r4 = (it1 % (kBM / 4)) * 4;
          const int i = t.ta * kBM + r4, j = j0 + c;
          float o[4] = {sum[e].x * p.out_scale, sum[e].y * p.out_scale, sum[e].z * p.out_scale, sum[e].w * p.out_scale};
          if (p.bias != nullptr) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              if (p.bias_on_a) { if (i + h < p.a_rows) o[h] += __bfloat162float(p.bias[i + h]); }
              else o[h] += __bfloat162float(p.bias[j]);
            }
          }
          __nv_bfloat16* dst = p.out + (long long)i * p.ldo_a + (long long)j * p.ldo_b;
          if (p.ldo_a == 1 && i + 4 <= p.a_rows && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
          } else {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              if (i + h < p.a_rows) dst[(long long)h * p.ldo_a] = __float2bfloat16(o[h]);
            }
          }
        }
      }
      // the last contributor to finish clears the counter for the next launch
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int prev = atomicAdd(&p.counters[t.counter], 0x10000);
        if ((prev >> 16) == t.nparts - 1) p.counters[t.counter] = 0;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if constexpr (LORA) {
    // the last CTA to finish clears the two counters for the next launch (every CTA is past its wait by then)
    if (lora && p.lora_inline_shrink && threadIdx.x == 0) {
      __threadfence();
      const int prev = atomicAdd(&p.lora_sync[0], 1);
      if (prev == (int)gridDim.x - 1) {
        p.lora_sync[0] = 0;
        p.lora_sync[1] = 0;
        __threadfence();
      }
    }
  }
}

// ---- LoRA shrink of a decode-sized step: v = A_cat(slot(t)) x[t] as matrix-vector products ---------------------------------
// The rows of a step are few and every one needs r * nparts dot products of length K with its own adapter's A_cat: bound by
// how fast A_cat streams in.  A CTA takes up to four rows of one table entry (they share the adapter, so A_cat is read once for
// them) and 16 of the rank rows, two per warp; a lane keeps 16 loads of 16 bytes in flight.  The results are written straight into the operand image of the entry (the layout the expand UMMAs of the GEMM read:
// [part][K slice][entry][48 rows][16 ranks], 32-byte swizzle); the CTAs that hold the first and the last row of an entry also
// clear the rows of the 16-aligned window that belong to neighbouring entries.
struct LoraShrinkRowsParams {
  const __nv_bfloat16* x;
  long long ldx;
  int T, K;
  const LoraTileG* tiles;
  int num_tiles;
  const __nv_bfloat16* arena;
  const int* slot_rank;
  const long long* slot_base;
  int num_slots;
  long long off_a;          // A_cat of the projection group and layer starts at slot_base + r * off_a (elements)
  int nparts;
  __nv_bfloat16* vimg;
};

LX_DEVICE float dot8_bf16(const uint4& a, const uint4& b) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 fa = __bfloat1622float2(pa[q]), fb = __bfloat1622float2(pb[q]);
    s = fmaf(fa.x, fb.x, s);
    s = fmaf(fa.y, fb.y, s);
  }
  return s;
}

constexpr int kShrinkRowsThreads = 256;
constexpr int kShrinkG = 4;             // rows of one entry that share a CTA
__global__ void __launch_bounds__(kShrinkRowsThreads) lora_shrink_rows_kernel(const LoraShrinkRowsParams p) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);                    // up to four rows of x, K bf16 each
  __shared__ int s_ent[5];                                           // entry index, slot, first row of the entry, its rows, group
  __shared__ int s_warp[8];
  __shared__ float s_v[3 * 64 * kShrinkG];
  const int tid = (int)threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_ent[0] = -1;
  // CTA b -> (entry, group of four rows): groups are numbered entry by entry (a prefix sum over the table).  The table is
  // written by copies that the stream orders before every kernel: it may be read before the wait below.
  int seen = 0;                                                      // groups of the entries before this round
  for (int lt0 = 0; lt0 < p.num_tiles; lt0 += kShrinkRowsThreads) {
    const int lt = lt0 + tid;
    int cnt = 0, slot = -1, row0 = 0, nr = 0;
    if (lt < p.num_tiles) {
      const LoraTileG e = p.tiles[lt];
      nr = min(min(e.nrows, 32), p.T - e.row0);
      slot = e.slot; row0 = e.row0;
      if (e.slot >= 0 && e.slot < p.num_slots && e.row0 >= 0 && nr > 0) cnt = (nr + kShrinkG - 1) / kShrinkG;
    }
    int incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    __syncthreads();                                                 // s_warp of the round before has been read
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = seen;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    const int first = before + incl - cnt;                           // this entry's groups are [first, first + cnt)
    const int b = (int)blockIdx.x;
    if (cnt > 0 && b >= first && b < first + cnt) {
      s_ent[0] = lt; s_ent[1] = slot; s_ent[2] = row0; s_ent[3] = nr; s_ent[4] = b - first;
    }
    for (int w = 0; w < 8; ++w) seen += s_warp[w];
  }
  __syncthreads();
  // Everything up to the wait reads only the table and the adapters, which no kernel of the step writes: it runs under the tail
  // of the kernel in front.  The first 8 loads per rank row are issued here, the rest of the two rows is pulled into L2.
  const int lt = s_ent[0];
  const int slot = lt >= 0 ? s_ent[1] : 0, row0 = s_ent[2], nrows = s_ent[3];
  const int t0 = row0 + s_ent[4] * kShrinkG;
  const int nt = min(kShrinkG, row0 + nrows - t0);                   // rows of this CTA: [t0, t0 + nt)
  const int r = lt >= 0 ? p.slot_rank[slot] : 0;
  const long long base = lt >= 0 ? p.slot_base[slot] : -1;
  const bool live = lt >= 0 && r > 0 && r <= 64 && (r & 15) == 0 && base >= 0;       // the GEMM skips the entry for the same reasons
  const int R = r * p.nparts;
  const int j_lo = (int)blockIdx.y * 16, j_hi = min(j_lo + 16, R);   // rank rows of this CTA, two per warp
  const bool work = live && j_lo < R;
  const int K8 = p.K >> 3;
  const int j = j_lo + 2 * warp;                                     // r is a multiple of 16: both rows exist
  const __nv_bfloat16* a_cat = p.arena + (work ? base + (long long)r * p.off_a : 0);
  const uint4* a0 = reinterpret_cast<const uint4*>(a_cat + (long long)j * p.K);
  const uint4* a1 = reinterpret_cast<const uint4*>(a_cat + (long long)(j + 1) * p.K);
  uint4 va[8], vb[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int k = lane + 32 * u;
    const bool in = work && k < K8;
    va[u] = in ? __ldg(a0 + k) : make_uint4(0, 0, 0, 0);
    vb[u] = in ? __ldg(a1 + k) : make_uint4(0, 0, 0, 0);
  }
  if (work) {
    for (int k = 256 + lane * 8; k < K8; k += 256) {               // one 128-byte line per lane and step
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a0 + k));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a1 + k));
    }
  }
  pdl_wait();
  if (!work) return;
  const int half = j_hi - j_lo;
  for (int q = 0; q < nt; ++q) {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x + (long long)(t0 + q) * p.ldx);
    for (int k = tid; k < K8; k += kShrinkRowsThreads) xs[q * K8 + k] = xg[k];
  }
  __syncthreads();
  {
    float s0[kShrinkG], s1[kShrinkG];
#pragma unroll
    for (int q = 0; q < kShrinkG; ++q) s0[q] = s1[q] = 0.f;
    for (int k0 = lane; k0 < K8; k0 += 32 * 8) {
      if (k0 != lane) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int k = k0 + 32 * u;
          va[u] = k < K8 ? __ldg(a0 + k) : make_uint4(0, 0, 0, 0);
          vb[u] = k < K8 ? __ldg(a1 + k) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + 32 * u;
        if (k < K8) {
#pragma unroll
          for (int q = 0; q < kShrinkG; ++q) {
            if (q < nt) {
              const uint4 xv = xs[q * K8 + k];
              s0[q] += dot8_bf16(va[u], xv);
              s1[q] += dot8_bf16(vb[u], xv);
            }
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < kShrinkG; ++q) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        s0[q] += __shfl_xor_sync(0xffffffffu, s0[q], d);
        s1[q] += __shfl_xor_sync(0xffffffffu, s1[q], d);
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int q = 0; q < kShrinkG; ++q) {
        s_v[q * 192 + j] = s0[q];
        s_v[q * 192 + j + 1] = s1[q];
      }
    }
  }
  __syncthreads();
  // image rows: 16 bytes = 8 ranks of one part; row c of the window holds row w0 + c of the step
  const int w0 = row0 & ~15;
  const int wn = ((row0 + nrows + 15) & ~15) - w0;
  const int nchunks = half >> 3;
  for (int u = tid; u < nchunks * nt; u += kShrinkRowsThreads) {
    const int q = u / nchunks, uc = u - q * nchunks;
    const int c = t0 + q - w0;
    const int j = j_lo + uc * 8;
    const int pp = j / r, i = j - pp * r;
    const int sl = i >> 4, ch = (i >> 3) & 1;
    __nv_bfloat16* img = p.vimg + ((long long)(pp * 4 + sl) * p.num_tiles + lt) * kLoraSliceElems;
    uint32_t pk[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) pk[h] = pack_bf16x2(s_v[q * 192 + j + 2 * h], s_v[q * 192 + j + 2 * h + 1]);
    *reinterpret_cast<uint4*>(img + c * 16 + ((ch ^ ((c >> 2) & 1)) << 3)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
  // rows of the window outside the entry: [0, z_lo) by the CTA of the first row, [z_hi, wn) by the CTA of the last one
  const int z_lo = (t0 == row0) ? row0 - w0 : 0;
  const int z_hi = (t0 + nt == row0 + nrows) ? row0 + nrows - w0 : wn;
  const int zrows = z_lo + (wn - z_hi);
  for (int u = tid; u < nchunks * zrows; u += kShrinkRowsThreads) {
    const int cz = u / nchunks, uc = u - cz * nchunks;
    const int row = cz < z_lo ? cz : z_hi + (cz - z_lo);
    const int j = j_lo + uc * 8;
    const int pp = j / r, i = j - pp * r;
    const int sl = i >> 4, ch = (i >> 3) & 1;
    __nv_bfloat16* img = p.vimg + ((long long)(pp * 4 + sl) * p.num_tiles + lt) * kLoraSliceElems;
    *reinterpret_cast<uint4*>(img + row * 16 + (ch << 3)) = make_uint4(0, 0, 0, 0);      // both chunks of a row are cleared: no swizzle needed
  }
}

static int launch_lora_shrink_rows(const LoraShrinkRowsParams& p, int max_rank, int num_sms, cudaStream_t stream) {
  const size_t smem = (size_t)p.K * 2 * kShrinkG;
  if (smem > 200 * 1024) return 1;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(lora_shrink_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int gy = (p.nparts * max_rank + 15) / 16;
  (void)num_sms;
  launch_pdl(lora_shrink_rows_kernel, dim3(p.T, gy), dim3(kShrinkRowsThreads), smem, stream, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
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

// The four arena-wide B_cat maps of a projection with N output features (see LoraBMaps).  0 on success.
static int make_lora_bmaps(LoraBMaps* out, const void* arena, long long arena_elems, int N) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr || (reinterpret_cast<uintptr_t>(arena) & 15) != 0) return -1;
  struct Key { const void* arena; long long elems; int N; };
  static Key keys[8];
  static LoraBMaps vals[8];
  static int used = 0, next = 0;
  for (int i = 0; i < used; ++i) {
    if (keys[i].arena == arena && keys[i].elems == arena_elems && keys[i].N == N) { *out = vals[i]; return 0; }
  }
  LoraBMaps bm{};
  for (int c = 0; c < 4; ++c) {
    const cuuint64_t r = 16 * (c + 1);
    cuuint64_t dims[3] = {r, (cuuint64_t)N, (cuuint64_t)(arena_elems / 8)};
    cuuint64_t strides[2] = {r * 2, 16};
    cuuint32_t box[3] = {16, (cuuint32_t)kBM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult rc = fn(&bm.m[c], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(arena), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return -2;
  }
  const int slot = used < 8 ? used++ : (next++ & 7);
  keys[slot] = Key{arena, arena_elems, N};
  vals[slot] = bm;
  *out = bm;
  return 0;
}

template <int BN, int STAGES, bool LORA>
static int launch_gemm_t(const CUtensorMap& ta, const CUtensorMap& tb, const LoraBMaps& bm, const GemmParams& p, int grid,
                         cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES, LORA>;
  // the shared-memory opt-in is a per-device attribute: one flag per device ordinal
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, STAGES, LORA>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return -(int)e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  launch_pdl(gemm_bf16_tcgen05_kernel<BN, STAGES, LORA>, dim3(grid), dim3(kGemmThreads), (size_t)S::kTotal, stream, ta, tb, bm, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e;
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  static const LoraBMaps none{};
  return launch_gemm_t<BN, STAGES, false>(ta, tb, none, p, grid, stream);
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

// Everything the LoRA part of a launch needs (see GemmParams): the table of the step, the slots' B_cat tensor maps for the
// expand stages, where the slots' blobs lie for the shrink kernel, and the scratch the operand images go to.
struct LxLoraFused {
  const void* tiles; int num_tiles;
  const void* slot_tmaps; int maps_per_slot, map_a, map_b;
  const int* slot_rank; const long long* slot_base; int num_slots;
  int nparts, n0, n1, layer, max_rank;
  void* vimg; long long vimg_bytes;
  int fence_maps;
  const void* arena; long long off_a;      // A_cat of the group and layer: arena + slot_base + rank * off_a (elements)
  long long off_b, arena_elems;            // B_cat likewise; the arena's size bounds the arena-wide maps
  int* sync;                               // two ints, zero before the first launch (see GemmParams::lora_sync)
};

static int gemm_impl(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                     long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                     int* status, int num_sms, int mode, int force_split, const LxLoraFused* lora, void* stream_) {
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
  const bool has_lora = (lora != nullptr && lora->tiles != nullptr && lora->num_tiles > 0);
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
  // operand).  Above that both plans are costed.  The LoRA stages are written for weights on M.
  bool swap;
  GemmPlan pl_swap{};
  if (mode == 1 || has_lora || (mode == 0 && T <= 128)) {
    swap = true;
  } else if (mode == 2) {
    swap = false;
  } else {
    pl_swap = choose_plan_swap(T, N, K, num_sms, usable_ws, have_counters, force_split & 0xffff, force_bn, sk_policy);
    swap = pl_swap.cost <= pl_tok.cost;
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
  if (has_lora) {
    p.lora_tiles = reinterpret_cast<const LoraTileG*>(lora->tiles);
    p.lora_num_tiles = lora->num_tiles;
    p.lora_slot_tmaps = reinterpret_cast<const CUtensorMap*>(lora->slot_tmaps);
    p.lora_maps_per_slot = lora->maps_per_slot; p.lora_map_a = lora->map_a; p.lora_map_b = lora->map_b;
    p.lora_slot_rank = lora->slot_rank; p.lora_slot_base = lora->slot_base; p.lora_num_slots = lora->num_slots;
    p.lora_nparts = lora->nparts; p.lora_n0 = lora->n0; p.lora_n1 = lora->n1; p.lora_layer = lora->layer;
    p.lora_vimg = reinterpret_cast<__nv_bfloat16*>(lora->vimg);
    p.lora_fence_maps = lora->fence_maps;
    p.lora_off_b = lora->off_b;
    LoraBMaps bm{};
    p.lora_arena_maps = (lora->arena_elems > 0 && make_lora_bmaps(&bm, lora->arena, lora->arena_elems, N) == 0) ? 1 : 0;
    {
      const char* e = getenv("LORAX_LORA_ARENA_MAPS");       // measurement only
      if (e && atoi(e) == 0) p.lora_arena_maps = 0;
    }
    {
      const char* e = getenv("LORAX_LORA_SKIP");       // measurement only
      p.lora_skip = e ? atoi(e) : 0;
    }
    p.lora_T = T;
    p.lora_off_a = lora->off_a;
    p.lora_arena = reinterpret_cast<const __nv_bfloat16*>(lora->arena);
    p.lora_x = reinterpret_cast<const __nv_bfloat16*>(x);
    p.lora_ldx = ldx;
    p.lora_max_r = lora->nparts * lora->max_rank;
    p.lora_sync = lora->sync;
    // the epilogue warps compute the shrink when every CTA of the launch is resident at once (the expand stages wait for all of
    // them) and the arena-wide maps give the entries their offsets; otherwise a launch in front does
    p.lora_inline_shrink = (lora->sync != nullptr && p.lora_arena_maps && pl.grid <= num_sms && !(p.lora_skip & 1)) ? 1 : 0;
    {
      const char* e = getenv("LORAX_LORA_INLINE_SHRINK");       // measurement only
      if (e && atoi(e) == 0) p.lora_inline_shrink = 0;
    }
    if (!(p.lora_skip & 1) && !p.lora_inline_shrink) {
      LoraShrinkRowsParams sp{};
      sp.x = reinterpret_cast<const __nv_bfloat16*>(x); sp.ldx = ldx; sp.T = T; sp.K = K;
      sp.tiles = p.lora_tiles; sp.num_tiles = p.lora_num_tiles;
      sp.arena = reinterpret_cast<const __nv_bfloat16*>(lora->arena);
      sp.slot_rank = lora->slot_rank; sp.slot_base = lora->slot_base; sp.num_slots = lora->num_slots;
      sp.off_a = lora->off_a; sp.nparts = lora->nparts;
      sp.vimg = p.lora_vimg;
      const int rc = launch_lora_shrink_rows(sp, lora->max_rank, num_sms, stream);
      if (rc != 0) return rc;
    }
    switch (template_bn(bn)) {
      case 16:  return launch_gemm_t<16, 8, true>(ta, tb, bm, p, pl.grid, stream);
      case 32:  return launch_gemm_t<32, 8, true>(ta, tb, bm, p, pl.grid, stream);
      case 64:  return launch_gemm_t<64, 8, true>(ta, tb, bm, p, pl.grid, stream);
      case 128: return launch_gemm_t<128, 6, true>(ta, tb, bm, p, pl.grid, stream);
      default:  return launch_gemm_t<256, 4, true>(ta, tb, bm, p, pl.grid, stream);
    }
  }
  switch (template_bn(bn)) {
    case 16:  return launch_gemm<16, 8>(ta, tb, p, pl.grid, stream);
    case 32:  return launch_gemm<32, 8>(ta, tb, p, pl.grid, stream);
    case 64:  return launch_gemm<64, 8>(ta, tb, p, pl.grid, stream);
    case 128: return launch_gemm<128, 6>(ta, tb, p, pl.grid, stream);
    default:  return launch_gemm<256, 4>(ta, tb, p, pl.grid, stream);
  }
}

// The plan the weights-on-M path would use for a shape: out5 = {token tile, classic split, whole tiles, stream-K CTAs, grid}.
int lx_gemm_plan(int T, int N, int K, int num_sms, long long ws_bytes, int force_split, int sk_policy, int* out5) {
  lx::GemmPlan pl = lx::choose_plan_swap(T, N, K, num_sms, ws_bytes, ws_bytes > 0, force_split & 0xffff, force_split >> 16, sk_policy);
  out5[0] = pl.bn; out5[1] = pl.split; out5[2] = pl.dp_tiles; out5[3] = pl.sk_ctas; out5[4] = pl.grid;
  return 0;
}

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N]).  `ldx`, `ldw`, `ldo` are row strides in elements.
// mode: low byte 0 = choose, 1 = force weights on the M side (small T), 2 = force activations on the M side; bits 8..9 the
// stream-K policy (0 by cost, 1 whole tiles only, 2 stream-K whenever a wave is partly filled).
// force_split: low 16 bits an exact classic K split, high 16 bits a forced token tile.
// Returns 0 or a negative error; device-side timeouts are reported through `status` (2 ints, zeroed by the caller).
int lx_gemm_bf16(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                 long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                 int* status, int num_sms, int mode, int force_split, void* stream_) {
  return gemm_impl(x, w, out, bias, T, N, K, ldx, ldw, ldo, out_scale, ws, ws_bytes, counters, status, num_sms, mode, force_split,
                   nullptr, stream_);
}

// The same GEMM with the multi-adapter LoRA of the step in the same launch: the epilogue warps compute the shrink during the
// first K loop, the delta is added by UMMAs into the accumulators of the base tiles (see the top of this file).  One launch
// replaces the shrink kernel, the base GEMM and the expand kernel of the reference (server/lorax_server/utils/layers.py:114-164).
// Returns 1 (nothing launched) when the step cannot be served this way: a part boundary that is not a multiple of 128, a rank
// above 64, or scratch too small for the table; the caller then runs shrink, GEMM and expand as separate launches.
int lx_gemm_bf16_lora(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                      long long ldw, long long ldo, void* ws, long long ws_bytes, int* counters, int* status, int num_sms,
                      const LxLoraFused* lora, void* stream_) {
  if (lora == nullptr || lora->tiles == nullptr || lora->num_tiles <= 0)
    return gemm_impl(x, w, out, bias, T, N, K, ldx, ldw, ldo, 1.f, ws, ws_bytes, counters, status, num_sms, 0, 0, nullptr, stream_);
  const bool bounds_ok = (lora->nparts == 1) || ((lora->n0 % lx::kBM) == 0 && (lora->nparts == 2 || (lora->n1 % lx::kBM) == 0));
  if (!bounds_ok || lora->max_rank > 64 || lora->max_rank <= 0 || lora->nparts < 1 || lora->nparts > 3 || N < lx::kBM) return 1;
  if ((long long)lora->num_tiles * lora->nparts * lx::kLoraImgElems * 2 > lora->vimg_bytes) return 1;
  if (lora->num_tiles > lx::kLoraMaxEntries || lora->arena == nullptr || (K & 7) != 0) return 1;
  return gemm_impl(x, w, out, bias, T, N, K, ldx, ldw, ldo, 1.f, ws, ws_bytes, counters, status, num_sms, 1, 0, lora, stream_);
}

int lx_lora_fused_desc_bytes() { return (int)sizeof(LxLoraFused); }

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
