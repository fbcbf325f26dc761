// Native executor for one decoder layer: issues every kernel of the attention half or of the MLP half from C++.
//
// The Python model code launches one kernel per ctypes call; an eager step (prefill, or a prefill riding along with a
// decode batch) is about 500 launches, which costs the host more than ten milliseconds whatever the GPU work is, and
// bounds the step time at tensor parallel 4 and 8.  Here Python describes the model once (LxModelDesc, one LxLayerDesc
// per layer) and a step once (LxStepDesc); each half of a layer is then ONE call that walks the same launchers
// (norm -> LoRA shrink -> GEMM -> LoRA expand -> RoPE + KV write -> attention -> ...).  The split into halves is where
// tensor parallelism needs its all-reduce, which stays with the caller.
//
// The reference runs this sequence as Python modules (server/lorax_server/models/custom_modeling/flash_llama_modeling.py:
// 262-330 attention, 364-410 MLP, 432-470 layer); there is no native counterpart there.
#include <cuda_runtime.h>

#include <cstdint>

extern "C" {

// launchers of this library (defined in the other translation units)
int lx_norm_residual(const void* x, void* residual, const void* w, const void* b, void* out, int T, int H, long long ldx,
                     long long ldr, long long ldo, float eps, float w_offset, float x_scale, int layernorm, void* stream);
int lx_rope_kvwrite(void* qkv, const int* positions, const float* cos_sin, void* kv_cache, const int* slots, int T, int nh,
                    int nkv, int d, int rot, int page, long long ldq, int apply_rope, void* stream);
int lx_act_mul(const void* in, void* out, int T, int I, long long ldi, long long ldo, int act, int gated, void* stream);
int lx_attn_decode(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                   void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                   float softcap, int nsplit, void* stream);
int lx_attn_prefill(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                    const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                    int nkv, int d, int window, float scale, float softcap, void* stream);
int lx_rope_kvwrite_kv8(void* qkv, const int* positions, const float* cos_sin, void* kv_cache, const int* slots, int T, int nh,
                        int nkv, int d, int rot, int page, long long ldq, int apply_rope, int kv_fp8, float k_scale, float v_scale,
                        void* stream);
int lx_attn_decode_kv8(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* ctx_lens,
                       void* out, long long ldo, float* part_o, float* part_lse, int T, int nh, int nkv, int d, int window, float scale,
                       float softcap, int nsplit, const float* alibi, float k_scale, float v_scale, void* stream);
int lx_attn_prefill_kv8(const void* q, long long ldq, const void* kv, const int* block_tables, int max_blocks, const int* cu_q,
                        const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo, int nh,
                        int nkv, int d, int window, float scale, float softcap, const float* alibi, float k_scale, float v_scale,
                        void* stream);
int lx_attn_prefill_tc_supported(int nh, int nkv, int d, long long ldq, long long ldo);
int lx_attn_prefill_tc(const void* q, long long ldq, int T, const void* kv, int num_blocks, const int* block_tables, int max_blocks,
                       const int* cu_q, const int* cache_lens, const int* tile_seq, const int* tile_q0, int num_tiles, void* out, long long ldo,
                       int nh, int nkv, int d, int window, float scale, float softcap, const float* alibi, int* status, void* stream);
int lx_lora_shrink(const void* x, long long ldx, const int* tok_slot, const void* arena, const long long* slot_base,
                   const int* slot_rank, int num_slots, long long unit_off, int nparts, float* v, int ldv, int T, int K,
                   int max_rank, int* status, void* stream);
int lx_lora_expand(const float* v, int ldv, const int* tok_slot, const void* arena, const long long* slot_base,
                   const int* slot_rank, int num_slots, long long unit_off, void* y, long long ldy, int T, int N, int n0, int n1,
                   int* status, void* stream);
int lx_lora_shrink_tc(const void* x, long long ldx, const void* tiles, int num_tiles, int max_tile_rows, const void* slot_tmaps,
                      int groups_per_slot, int group, const int* slot_rank, int num_slots, int nparts, int layer, float* v, int ldv,
                      long long v_split_stride, int ksplit, float* v_final, int* counters, int num_counters, int T, int K, int max_rank,
                      int* status, void* stream);
int lx_lora_expand_tiled(const float* v, int ldv, long long v_split_stride, int ksplit, const void* tiles, int num_tiles,
                         int max_tile_rows, const void* arena, const long long* slot_base, const int* slot_rank, int num_slots,
                         long long unit_off, void* y, long long ldy, int T, int N, int n0, int n1, int* status, void* stream);
int lx_gemm_bf16(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                 long long ldw, long long ldo, float out_scale, void* ws, long long ws_bytes, int* counters,
                 int* status, int num_sms, int mode, int force_split, void* stream_);
struct LxLoraFused {
  const void* tiles; int num_tiles;
  const void* slot_tmaps; int maps_per_slot, map_a, map_b;
  const int* slot_rank; const long long* slot_base; int num_slots;
  int nparts, n0, n1, layer, max_rank;
  void* vimg; long long vimg_bytes;
  int fence_maps;
  const void* arena; long long off_a;
  long long off_b, arena_elems;
  int* sync;
};
int lx_gemm_bf16_lora(const void* x, const void* w, void* out, const void* bias, int T, int N, int K, long long ldx,
                      long long ldw, long long ldo, void* ws, long long ws_bytes, int* counters, int* status, int num_sms,
                      const LxLoraFused* lora, void* stream_);
int lx_allreduce_sym(const unsigned long long* peer_ptrs, int rank, int world, long long in_off, long long out_off, long long cnt_off,
                     long long n_elems, int* state, int* status, void* stream);

// The two-shot all-reduce of a tensor-parallel group as the layer loop needs it: every partial sum is written into the input
// area of the rank's symmetric buffer and the reduced activations are read from its output area.
struct LxAllReduce {
  const unsigned long long* peer_ptrs;   // base of every rank's symmetric buffer
  long long in_off, out_off, cnt_off;    // byte offsets inside the buffer
  int* state;                            // two device ints (launch counter, finished blocks)
  int* status;
  int rank, world;
};

// One LoRA site of a layer (QKV, O, gate_up, down): where its A_cat / B_cat sit inside every adapter blob.
struct LxLoraSite {
  long long off_a, off_b;        // in units (multiply by the slot's rank)
  int nparts, n0, n1;            // parts of the fused projection and their boundaries along N
  int tmap_group;                // index of the site's tensor map inside a slot's map family
  int enabled;
  int pad_;
};

struct LxLayerDesc {
  const void* input_norm_w; const void* input_norm_b;
  const void* post_norm_w;  const void* post_norm_b;
  const void* qkv_w; const void* qkv_b;
  const void* o_w;   const void* o_b;
  const void* gate_up_w; const void* gate_up_b;
  const void* down_w;    const void* down_b;
  long long ld_qkv, ld_o, ld_gate_up, ld_down;     // row strides of the weights (elements)
  void* kv_cache;
  LxLoraSite lora[4];
  int layer_index;               // third coordinate of the adapter tensor maps
  int window;                    // sliding window of this layer (0 = none)
  float k_scale, v_scale;        // e4m3 cache: stored value * scale is the key / value (see LxModelDesc::kv_fp8)
};

struct LxModelDesc {
  int H, nh, nkv, d, inter, rot, page, apply_rope, act, gated, layernorm, pad0_;
  int n_qkv, n_o_in, n_gate_up, n_down_in;       // GEMM shapes: qkv out, O in (= nh * d), gate_up out, down in
  float eps, norm_offset, attn_scale, softcap;
  const float* cos_sin;
  // scratch shared by the kernels
  void* gemm_ws; long long gemm_ws_bytes; int* gemm_counters; int* status; int num_sms; int pad1_;
  float* lora_v3; long long v3_plane_stride; int v3_planes; int ldv; float* lora_v; int* lora_counters; int n_lora_counters; int pad2_;
  float* attn_part_o; float* attn_part_lse; int attn_splits; int attn_part_tokens;
  // adapters
  const void* arena; const long long* slot_base; const int* slot_rank; const void* slot_tmaps;
  int num_slots, max_rank, groups_per_slot, fused_lora;      // fused_lora: rows up to which LoRA rides inside the GEMM launch (0: never)
  // scratch of the GEMM that carries LoRA in its own launch
  void* lora_vimg; long long lora_vimg_bytes; long long arena_elems; int* lora_sync; int lora_fence_maps;
  int tc_prefill, kv_blocks;     // tensor-core prefill attention where the shape allows; blocks of the paged cache
  int kv_fp8, pad3_;             // the cache holds e4m3 bytes
};

struct LxStepDesc {
  int T, n_decode;               // rows [0, n_decode) are decode rows, the rest prefill tokens
  const int* positions; const int* slots;
  const int* dec_block_tables; const int* ctx_lens; int dec_max_blocks; int nsplit;
  const int* block_tables; const int* cu_q; const int* cache_lens; const int* tile_seq; const int* tile_q0;
  int max_blocks, n_attn_tiles;
  const int* tok_slot;           // nullptr: no adapter in this step
  const void* lora_tiles;        // nullptr: rows are not grouped by adapter, use the per-token kernels
  int num_tiles, max_tile_rows;
  int live_tiles, pad5_;         // live entries of the table (0: all)
  // activations of the step (allocated by the caller, reused by every layer)
  void* normed; void* qkv; void* attn; void* gate_up; void* act;
};

}  // extern "C"

namespace {

#define LX_TRY(expr)            \
  do {                          \
    int rc_ = (expr);           \
    if (rc_ != 0) return rc_;   \
  } while (0)

// y[T, N] = x[T, K] w^T (+ bias) (+ LoRA delta of the site)
int linear_with_lora(const LxModelDesc& m, const LxLayerDesc& l, const LxStepDesc& s, int site_idx, const void* x, long long ldx,
                     const void* w, long long ldw, const void* bias, void* y, long long ldy, int N, int K, void* stream) {
  const LxLoraSite& site = l.lora[site_idx];
  const bool lora = s.tok_slot != nullptr && site.enabled && m.max_rank > 0 && (s.lora_tiles == nullptr || s.num_tiles > 0);
  if (lora && s.lora_tiles != nullptr && s.T <= m.fused_lora && s.max_tile_rows <= 32) {
    // one launch: shrink on the epilogue warps, base tiles, expand UMMAs
    LxLoraFused f{};
    f.tiles = s.lora_tiles; f.num_tiles = s.num_tiles;
    f.slot_tmaps = m.slot_tmaps; f.maps_per_slot = m.groups_per_slot; f.map_a = site.tmap_group; f.map_b = m.groups_per_slot / 2 + site.tmap_group;
    f.slot_rank = m.slot_rank; f.slot_base = m.slot_base; f.num_slots = m.num_slots;
    f.nparts = site.nparts; f.n0 = site.n0; f.n1 = site.n1; f.layer = l.layer_index; f.max_rank = m.max_rank;
    f.vimg = m.lora_vimg; f.vimg_bytes = m.lora_vimg_bytes; f.fence_maps = m.lora_fence_maps;
    f.arena = m.arena; f.off_a = site.off_a; f.off_b = site.off_b; f.arena_elems = m.arena_elems; f.sync = m.lora_sync;
    const int rc = lx_gemm_bf16_lora(x, w, y, bias, s.T, N, K, ldx, ldw, ldy, m.gemm_ws, m.gemm_ws_bytes, m.gemm_counters, m.status, m.num_sms,
                                     &f, stream);
    if (rc != 1) return rc;          // 1: this step does not fit the fused launch, use the separate kernels below
  }
  if (lora) {
    if (s.lora_tiles != nullptr) {
      const int kblocks = (K + 63) / 64;
      const int chunks = (site.nparts * m.max_rank + 127) / 128;
      int ksplit = (2 * m.num_sms) / (s.num_tiles * chunks);       // one wave of CTAs (two per SM), see ops/native.py
      if (ksplit > kblocks / 8) ksplit = kblocks / 8;
      if (ksplit > m.v3_planes) ksplit = m.v3_planes;
      if (ksplit < 1) ksplit = 1;
      LX_TRY(lx_lora_shrink_tc(x, ldx, s.lora_tiles, s.num_tiles, s.max_tile_rows, m.slot_tmaps, m.groups_per_slot, site.tmap_group,
                               m.slot_rank, m.num_slots, site.nparts, l.layer_index, m.lora_v3, m.ldv, m.v3_plane_stride, ksplit,
                               m.lora_v, m.lora_counters, m.n_lora_counters, s.T, K, m.max_rank, m.status, stream));
    } else {
      LX_TRY(lx_lora_shrink(x, ldx, s.tok_slot, m.arena, m.slot_base, m.slot_rank, m.num_slots, site.off_a, site.nparts, m.lora_v, m.ldv,
                            s.T, K, m.max_rank, m.status, stream));
    }
  }
  LX_TRY(lx_gemm_bf16(x, w, y, bias, s.T, N, K, ldx, ldw, ldy, 1.f, m.gemm_ws, m.gemm_ws_bytes, m.gemm_counters, m.status, m.num_sms, 0, 0,
                      stream));
  if (lora) {
    if (s.lora_tiles != nullptr) {
      LX_TRY(lx_lora_expand_tiled(m.lora_v, m.ldv, 0, 1, s.lora_tiles, s.num_tiles, s.max_tile_rows, m.arena, m.slot_base, m.slot_rank,
                                  m.num_slots, site.off_b, y, ldy, s.T, N, site.n0, site.n1, m.status, stream));
    } else {
      LX_TRY(lx_lora_expand(m.lora_v, m.ldv, s.tok_slot, m.arena, m.slot_base, m.slot_rank, m.num_slots, site.off_b, y, ldy, s.T, N,
                            site.n0, site.n1, m.status, stream));
    }
  }
  return 0;
}

}  // namespace

extern "C" {

int lx_layer_desc_bytes() { return (int)sizeof(LxLayerDesc); }
int lx_model_desc_bytes() { return (int)sizeof(LxModelDesc); }
int lx_step_desc_bytes() { return (int)sizeof(LxStepDesc); }

// Attention half: normed = norm(x_in * x_scale + residual) (residual updated in place; x_in == nullptr: normed =
// norm(residual)), QKV projection, RoPE + KV write, attention, O projection -> out [T, H] (this rank's partial sum
// under tensor parallelism).
int lx_layer_attention(const LxModelDesc* m, const LxLayerDesc* l, const LxStepDesc* s, const void* x_in, void* residual, float x_scale,
                       void* out, void* stream) {
  const int T = s->T, H = m->H;
  if (T <= 0) return 0;
  if (x_in != nullptr) {
    LX_TRY(lx_norm_residual(x_in, residual, l->input_norm_w, l->input_norm_b, s->normed, T, H, H, H, H, m->eps, m->norm_offset, x_scale,
                            m->layernorm, stream));
  } else {
    LX_TRY(lx_norm_residual(residual, nullptr, l->input_norm_w, l->input_norm_b, s->normed, T, H, H, 0, H, m->eps, m->norm_offset, 1.f,
                            m->layernorm, stream));
  }
  LX_TRY(linear_with_lora(*m, *l, *s, 0, s->normed, H, l->qkv_w, l->ld_qkv, l->qkv_b, s->qkv, m->n_qkv, m->n_qkv, H, stream));
  LX_TRY(lx_rope_kvwrite_kv8(s->qkv, s->positions, m->cos_sin, l->kv_cache, s->slots, T, m->nh, m->nkv, m->d, m->rot, m->page, m->n_qkv,
                             m->apply_rope, m->kv_fp8, l->k_scale, l->v_scale, stream));
  const int nd = s->n_decode;
  const long long ldq = m->n_qkv, lda = m->n_o_in;
  char* q = reinterpret_cast<char*>(s->qkv);
  char* a = reinterpret_cast<char*>(s->attn);
  if (nd > 0) {
    int nsplit = s->nsplit;
    if (nsplit > m->attn_splits) nsplit = m->attn_splits;
    if (nd > m->attn_part_tokens || nsplit < 1) nsplit = 1;
    if (m->kv_fp8) {
      LX_TRY(lx_attn_decode_kv8(q, ldq, l->kv_cache, s->dec_block_tables, s->dec_max_blocks, s->ctx_lens, a, lda, m->attn_part_o,
                                m->attn_part_lse, nd, m->nh, m->nkv, m->d, l->window, m->attn_scale, m->softcap, nsplit, nullptr,
                                l->k_scale, l->v_scale, stream));
    } else {
      LX_TRY(lx_attn_decode(q, ldq, l->kv_cache, s->dec_block_tables, s->dec_max_blocks, s->ctx_lens, a, lda, m->attn_part_o, m->attn_part_lse,
                            nd, m->nh, m->nkv, m->d, l->window, m->attn_scale, m->softcap, nsplit, stream));
    }
  }
  if (T > nd) {
    if (m->kv_fp8) {
      // the tensor-core kernel reads bf16 pages by TMA; the e4m3 cache goes through the kernel that expands pages in shared memory
      LX_TRY(lx_attn_prefill_kv8(q + (long long)nd * ldq * 2, ldq, l->kv_cache, s->block_tables, s->max_blocks, s->cu_q, s->cache_lens,
                                 s->tile_seq, s->tile_q0, s->n_attn_tiles, a + (long long)nd * lda * 2, lda, m->nh, m->nkv, m->d, l->window,
                                 m->attn_scale, m->softcap, nullptr, l->k_scale, l->v_scale, stream));
    } else if (m->tc_prefill && lx_attn_prefill_tc_supported(m->nh, m->nkv, m->d, ldq, lda)) {
      LX_TRY(lx_attn_prefill_tc(q + (long long)nd * ldq * 2, ldq, T - nd, l->kv_cache, m->kv_blocks, s->block_tables, s->max_blocks, s->cu_q,
                                s->cache_lens, s->tile_seq, s->tile_q0, s->n_attn_tiles, a + (long long)nd * lda * 2, lda, m->nh, m->nkv, m->d,
                                l->window, m->attn_scale, m->softcap, nullptr, m->status, stream));
    } else {
      LX_TRY(lx_attn_prefill(q + (long long)nd * ldq * 2, ldq, l->kv_cache, s->block_tables, s->max_blocks, s->cu_q, s->cache_lens, s->tile_seq,
                             s->tile_q0, s->n_attn_tiles, a + (long long)nd * lda * 2, lda, m->nh, m->nkv, m->d, l->window, m->attn_scale,
                             m->softcap, stream));
    }
  }
  return linear_with_lora(*m, *l, *s, 1, s->attn, lda, l->o_w, l->ld_o, l->o_b, out, H, H, m->n_o_in, stream);
}

// MLP half: normed = norm(x_in * x_scale + residual) (residual updated), gate_up projection, activation (* up), down
// projection -> out [T, H] (partial under tensor parallelism).
int lx_layer_mlp(const LxModelDesc* m, const LxLayerDesc* l, const LxStepDesc* s, const void* x_in, void* residual, float x_scale, void* out,
                 void* stream) {
  const int T = s->T, H = m->H;
  if (T <= 0) return 0;
  LX_TRY(lx_norm_residual(x_in, residual, l->post_norm_w, l->post_norm_b, s->normed, T, H, H, H, H, m->eps, m->norm_offset, x_scale,
                          m->layernorm, stream));
  LX_TRY(linear_with_lora(*m, *l, *s, 2, s->normed, H, l->gate_up_w, l->ld_gate_up, l->gate_up_b, s->gate_up, m->n_gate_up, m->n_gate_up, H,
                          stream));
  LX_TRY(lx_act_mul(s->gate_up, s->act, T, m->inter, m->n_gate_up, m->inter, m->act, m->gated, stream));
  return linear_with_lora(*m, *l, *s, 3, s->act, m->inter, l->down_w, l->ld_down, l->down_b, out, H, H, m->n_down_in, stream);
}

int lx_allreduce_desc_bytes() { return (int)sizeof(LxAllReduce); }

// Every layer of the model in one call: attention half, all-reduce, MLP half, all-reduce (the collectives only with `ar`, i.e.
// under tensor parallelism).  `residual` [T, H] holds the embedded tokens on entry and the residual stream on return; the output
// of the last MLP half that still has to be added to it is at `*pending_out` (inside the symmetric buffer with `ar`, else `scratch`,
// which must hold T * H elements).
int lx_run_layers(const LxModelDesc* m, const LxLayerDesc* layers, int n_layers, const LxStepDesc* s, void* residual, float x_scale,
                  const LxAllReduce* ar, void* scratch, void** pending_out, void* stream) {
  const long long n = (long long)s->T * m->H;
  unsigned char* base = ar ? reinterpret_cast<unsigned char*>(ar->peer_ptrs[ar->rank]) : nullptr;
  void* part = ar ? static_cast<void*>(base + ar->in_off) : scratch;      // where a half writes its (partial) result
  void* full = ar ? static_cast<void*>(base + ar->out_off) : scratch;     // where the next half reads the complete one
  const void* pending = nullptr;
  for (int li = 0; li < n_layers; ++li) {
    LX_TRY(lx_layer_attention(m, &layers[li], s, pending, residual, x_scale, part, stream));
    if (ar) LX_TRY(lx_allreduce_sym(ar->peer_ptrs, ar->rank, ar->world, ar->in_off, ar->out_off, ar->cnt_off, n, ar->state, ar->status, stream));
    LX_TRY(lx_layer_mlp(m, &layers[li], s, full, residual, x_scale, part, stream));
    if (ar) LX_TRY(lx_allreduce_sym(ar->peer_ptrs, ar->rank, ar->world, ar->in_off, ar->out_off, ar->cnt_off, n, ar->state, ar->status, stream));
    pending = full;
  }
  *pending_out = const_cast<void*>(pending);
  return 0;
}

}  // extern "C"
