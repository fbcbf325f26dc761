"""Weight-only quantisation: checkpoint layouts (GPTQ, AWQ), the resident packed layout, the on-load quantisers, GPTQ itself,
loading a packed checkpoint into the decoder, and (on a GPU) the expansion and 4-bit tensor-core kernels against the fp32
reference.  The reference covers the same ground with per-format extensions (server/lorax_server/layers/linear.py:93-181,
utils/gptq/quantize.py, utils/weights.py:98-234)."""

import json

import pytest
import torch

from lorax_b200 import config as cfgs
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.models.loading import export_hf_state_dict
from lorax_b200.utils import quant_formats as qf
from lorax_b200.utils.weights import InMemoryWeights, checkpoint_quantization


def _naive_gptq_dequant(qweight, qzeros, scales, g_idx, bits):
    """The AutoGPTQ layout, element by element."""
    per = 32 // bits
    Kp, N = qweight.shape
    K = Kp * per
    mask = (1 << bits) - 1
    w = torch.zeros(K, N)
    for k in range(K):
        for n in range(N):
            q = (int(qweight[k // per, n]) >> (bits * (k % per))) & mask
            z = ((int(qzeros[int(g_idx[k]), n // per]) >> (bits * (n % per))) & mask) + 1
            w[k, n] = float(scales[int(g_idx[k]), n]) * (q - z)
    return w.t()


def _naive_awq_dequant(qweight, qzeros, scales, group):
    K, Np = qweight.shape
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    w = torch.zeros(K, Np * 8)
    for k in range(K):
        for c in range(Np):
            for i in range(8):
                n = c * 8 + order[i]
                q = (int(qweight[k, c]) >> (4 * i)) & 15
                z = (int(qzeros[k // group, c]) >> (4 * i)) & 15
                w[k, n] = float(scales[k // group, n]) * (q - z)
    return w.t()


def test_resident_layout_roundtrip_and_slices():
    torch.manual_seed(0)
    for bits in (2, 4, 8):
        q = torch.randint(0, 1 << bits, (24, 256), dtype=torch.int32)
        assert torch.equal(qf.unpack_codes(qf.pack_codes(q, bits), bits, 256), q)
    # the 4-bit interleave: nibble i of every 32-bit word holds k = 8 * word + NIBBLE_K[i]
    q = torch.arange(16, dtype=torch.int32).view(1, 16) % 16
    word = int.from_bytes(bytes(qf.pack_codes(q, 4)[0, :4].tolist()), "little")
    assert [(word >> (4 * i)) & 15 for i in range(8)] == [0, 2, 4, 6, 1, 3, 5, 7]
    w = torch.randn(64, 512)
    g = qf.quantize_rtn(w, 4, 128)
    d = qf.dequantize(g)
    assert torch.equal(qf.dequantize(g[16:48]), d[16:48])
    assert torch.equal(qf.dequantize(g[:, 128:384]), d[:, 128:384])
    assert torch.equal(qf.dequantize(qf.cat_rows([g[:16], g[16:]])), d)
    with pytest.raises(ValueError):
        g[:, 64:192]


def test_gptq_and_awq_checkpoint_layouts_match_their_specification():
    torch.manual_seed(1)
    N, K, group = 16, 64, 32
    q = torch.randint(0, 16, (N, K), dtype=torch.int32)
    s = (torch.rand(N, K // group) * 0.1 + 0.01).to(torch.float16).float()
    z = torch.randint(1, 16, (N, K // group)).float()
    t = qf.gptq_pack(q, s, z, 4, group)
    assert t["qweight"].shape == (K // 8, N) and t["qzeros"].shape == (K // group, N // 8) and t["qweight"].dtype == torch.int32
    want = _naive_gptq_dequant(t["qweight"], t["qzeros"], t["scales"], t["g_idx"], 4)
    packed, dense = qf.from_checkpoint(t, "gptq", 4, group)
    assert packed is not None and torch.allclose(dense.float(), want, atol=2e-3)
    assert torch.allclose(qf.dequantize(packed), want, atol=1e-6)
    # act-order: groups are no longer runs of consecutive inputs -> the packed form keeps the columns sorted by group and the
    # order they came from; expanded, it honours g_idx
    perm = torch.randperm(K)
    t2 = dict(t)
    t2["g_idx"] = (perm // group).to(torch.int32)
    want2 = _naive_gptq_dequant(t2["qweight"], t2["qzeros"], t2["scales"], t2["g_idx"], 4)
    packed2, dense2 = qf.from_checkpoint(t2, "gptq", 4, group)
    assert packed2 is not None and packed2.perm is not None and sorted(packed2.perm.tolist()) == list(range(K))
    assert torch.allclose(dense2.float(), want2, atol=2e-3) and torch.allclose(qf.dequantize(packed2), want2, atol=1e-6)
    x = torch.randn(5, K)
    assert torch.allclose(x[:, packed2.perm.long()] @ qf.dequantize(qf.GroupQuantWeight(
        packed2.codes, packed2.sz, 4, group, packed2.shape)).t(), x @ want2.t(), atol=1e-4)
    with pytest.raises(ValueError):
        packed2.cols(0, group)
    # groups of unequal size have no packed form
    t3 = dict(t)
    t3["g_idx"] = torch.cat([torch.zeros(group + 8), torch.ones(K - group - 8)]).to(torch.int32)
    packed3, dense3 = qf.from_checkpoint(t3, "gptq", 4, group)
    assert packed3 is None
    assert torch.allclose(dense3.float(), _naive_gptq_dequant(t3["qweight"], t3["qzeros"], t3["scales"], t3["g_idx"], 4), atol=2e-3)
    # 8-bit GPTQ and the v2 zero convention
    q8 = torch.randint(0, 256, (N, K), dtype=torch.int32)
    z8 = torch.randint(1, 255, (N, K // group)).float()
    t8 = qf.gptq_pack(q8, s, z8, 8, group)
    p8, _ = qf.from_checkpoint(t8, "gptq", 8, group)
    assert torch.allclose(qf.dequantize(p8), _naive_gptq_dequant(t8["qweight"], t8["qzeros"], t8["scales"], t8["g_idx"], 8), atol=1e-5)
    tv2 = qf.gptq_pack(q, s, z, 4, group, zero_offset=0)
    pv2, _ = qf.from_checkpoint(tv2, "gptq", 4, group, zero_offset=0)
    assert torch.equal(qf.dequantize(pv2), qf.dequantize(packed))
    # AWQ
    ta = qf.awq_pack(q, s, z)
    assert ta["qweight"].shape == (K, N // 8)
    pa, _ = qf.from_checkpoint(ta, "awq", 4, group, zero_offset=0)
    assert torch.allclose(qf.dequantize(pa), _naive_awq_dequant(ta["qweight"], ta["qzeros"], ta["scales"], group), atol=1e-6)


@pytest.mark.parametrize("method,bound", [("int4", 0.12), ("gptq", 0.12), ("awq", 0.12), ("eetq", 0.012), ("bitsandbytes", 0.012),
                                          ("bitsandbytes-nf4", 0.11), ("bitsandbytes-fp4", 0.15), ("hqq-4bit", 0.10),
                                          ("hqq-3bit", 0.21), ("hqq-2bit", 0.50)])
def test_on_load_quantisers_error_bounds(method, bound):
    torch.manual_seed(2)
    w = torch.randn(48, 512) * 0.05
    g = qf.quantize_weight(w, method)
    err = ((qf.dequantize(g) - w).norm() / w.norm()).item()
    assert err < bound, (method, err)
    x = torch.randn(7, 512)
    from lorax_b200.ops import reference as ref
    y = ref.gemm_wq(x, g, bias=torch.ones(48))
    assert torch.allclose(y, x @ qf.dequantize(g).t() + 1.0, atol=1e-4)


def test_hqq_beats_round_to_nearest_at_low_bits():
    torch.manual_seed(3)
    w = torch.randn(64, 512) * 0.05
    w[:, ::37] *= 6.0                                   # outliers: where a refined zero point pays
    for bits in (3, 2):
        hqq = qf.dequantize(qf.quantize_hqq(w, bits, 64))
        maxq = (1 << bits) - 1
        x = w.view(64, -1, 64)
        lo, hi = x.amin(-1, keepdim=True), x.amax(-1, keepdim=True)
        sc = (hi - lo) / maxq
        rtn = ((torch.clamp(torch.round((x - lo) / sc), 0, maxq)) * sc + lo).view(64, 512)
        # the l_p (p < 1) objective HQQ minimises
        assert (hqq - w).abs().pow(0.7).sum() < (rtn - w).abs().pow(0.7).sum()


def test_three_bit_gptq_checkpoints_load_into_the_four_bit_layout():
    """3-bit GPTQ packs 32 codes into three int32 as one bit stream (codes 10 and 21 straddle words; AutoGPTQ's `pack` writes the
    low bits of a straddling code into the top of one word and the rest into the bottom of the next).  The codes and zero points
    are exact in the resident 4-bit layout, so the layer is served packed."""
    torch.manual_seed(7)
    N, K, group = 32, 128, 64
    q = torch.randint(0, 8, (N, K), dtype=torch.int32)
    s = (torch.rand(N, K // group) * 0.1 + 0.01).to(torch.float16).float()
    z = torch.randint(1, 8, (N, K // group)).float()
    t = qf.gptq_pack(q, s, z, 3, group)
    assert t["qweight"].shape == (K * 3 // 32, N) and t["qweight"].dtype == torch.int32
    # the packing against AutoGPTQ's word-by-word description, for one column
    col = q[5].tolist()
    w0 = sum(col[j] << (3 * j) for j in range(10)) | ((col[10] << 30) & 0xFFFFFFFF)
    w1 = ((col[10] >> 2) & 1) | sum(col[11 + j] << (3 * j + 1) for j in range(10)) | ((col[21] << 31) & 0xFFFFFFFF)
    w2 = ((col[21] >> 1) & 3) | sum(col[22 + j] << (3 * j + 2) for j in range(10))
    got = [int(v) & 0xFFFFFFFF for v in t["qweight"][:3, 5]]
    assert got == [w0 & 0xFFFFFFFF, w1 & 0xFFFFFFFF, w2 & 0xFFFFFFFF]
    uq, us, uz = qf.gptq_unpack(t["qweight"], t["qzeros"], t["scales"], 3)
    assert torch.equal(uq, q) and torch.equal(uz, z) and torch.allclose(us, s, atol=1e-3)
    packed, dense = qf.from_checkpoint(t, "gptq", 3, group)
    want = (q.float() - z.repeat_interleave(group, 1)) * s.repeat_interleave(group, 1)
    assert packed is not None and packed.bits == 4
    assert torch.allclose(dense.float(), want, atol=2e-3) and torch.allclose(qf.dequantize(packed), want, atol=1e-6)


def test_gptq_compensates_rounding_error_through_the_hessian():
    torch.manual_seed(4)
    w = torch.randn(64, 256)
    X = torch.randn(4096, 64) @ torch.randn(64, 256) + 0.3 * torch.randn(4096, 256)     # correlated inputs
    Q, sc, zp = qf.gptq_quantize(w, X.t() @ X, bits=4, group=128)
    wg = qf.dequantize(qf.make_weight(Q, sc, zp, 4, 128))
    wr = qf.dequantize(qf.quantize_rtn(w, 4, 128))
    ref = X @ w.t()
    e_g = ((X @ wg.t() - ref).norm() / ref.norm()).item()
    e_r = ((X @ wr.t() - ref).norm() / ref.norm()).item()
    assert e_g < 0.6 * e_r, (e_g, e_r)
    assert int(Q.min()) >= 0 and int(Q.max()) <= 15


def _tiny(vocab=512):
    cfg = cfgs.tiny_llama(vocab)
    cfg.intermediate_size = 768
    return cfg


def _forward(model, ids):
    """Logits of every prompt position through the model's own forward pass."""
    from lorax_b200.runtime.kv_cache import KVCache
    from lorax_b200.runtime.runner import ModelRunner, PrefillItem
    kv = KVCache(model.config.num_hidden_layers, 16, model.nkv, model.d, model.dtype, model.device)
    r = ModelRunner(model, kv, max_batch=2, max_seq_tokens=128, max_prefill_tokens=256, use_graphs=False)
    return r.prefill([PrefillItem(ids, 0, [1, 2, 3, 4], all_logprobs=True)])[2]


def test_gptq_checkpoint_loads_packed_and_matches_its_dense_expansion(tmp_path):
    cfg = _tiny()
    dense_model = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=5, std=0.05)
    sd = export_hf_state_dict(dense_model)
    qsd, deq = {}, {}
    for k, t in sd.items():
        if k.endswith("_proj.weight"):
            g = qf.quantize_rtn(t, 4, 128)
            q = qf.unpack_codes(g.codes, 4, t.shape[1])
            for n, v in qf.gptq_pack(q, g.sz[..., 0].float(), g.sz[..., 1].float(), 4, 128).items():
                qsd[k[:-6] + n] = v
            deq[k] = qf.dequantize(g)
        else:
            qsd[k] = t
            deq[k] = t
    w = InMemoryWeights(qsd, dtype=torch.float32)
    w.quant = {"quant_method": "gptq", "bits": 4, "group_size": 128, "zero_offset": 1}
    mq = DecoderModel.from_weights(cfg, w, torch.device("cpu"), torch.float32)
    assert mq.quantized == "gptq"
    assert all(isinstance(getattr(lw, n), qf.GroupQuantWeight) for lw in mq.layers for n in ("qkv_w", "o_w", "gate_up_w", "down_w"))
    md = DecoderModel.from_weights(cfg, InMemoryWeights(deq, dtype=torch.float32), torch.device("cpu"), torch.float32)
    ids = list(range(3, 40))
    a, b = _forward(mq, ids), _forward(md, ids)
    assert torch.allclose(a, b, atol=2e-4), (a - b).abs().max()
    # the same checkpoint expanded on load (another scheme was asked for)
    w2 = InMemoryWeights(qsd, dtype=torch.float32)
    w2.quant, w2.keep_packed = w.quant, False
    m2 = DecoderModel.from_weights(cfg, w2, torch.device("cpu"), torch.float32)
    assert m2.quantized is None and torch.allclose(_forward(m2, ids), b, atol=2e-3)
    # and the config files that announce such a checkpoint
    (tmp_path / "quantize_config.json").write_text(json.dumps({"bits": 4, "group_size": 128, "desc_act": False}))
    assert checkpoint_quantization(tmp_path) == {"quant_method": "gptq", "bits": 4, "group_size": 128, "zero_offset": 1, "desc_act": False}
    assert checkpoint_quantization(tmp_path, {"quantization_config": {"quant_method": "awq", "bits": 4, "group_size": 64}})["zero_offset"] == 0
    assert checkpoint_quantization(tmp_path, {"quantization_config": {"quant_method": "fp8"}}) is None


def test_act_order_gptq_checkpoint_is_served_packed():
    """`desc_act` checkpoints: every projection stays packed (columns sorted by group, activations gathered in that order in
    front of the GEMM) and the model's logits equal those of the checkpoint expanded to dense matrices."""
    cfg = _tiny()
    dense_model = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=7, std=0.05)
    sd = export_hf_state_dict(dense_model)
    gen = torch.Generator().manual_seed(3)
    orders = {}                                            # one column order per layer input, as the Hessian of that input gives
    qsd, deq = {}, {}
    for k, t in sd.items():
        if not k.endswith("_proj.weight"):
            qsd[k] = deq[k] = t
            continue
        site = k.rsplit(".", 3)[0] + (".in_h" if any(n in k for n in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")) else k)
        K = t.shape[1]
        perm = orders.setdefault((site, K), torch.randperm(K, generator=gen))
        g = qf.quantize_rtn(t[:, perm].contiguous(), 4, 128)
        codes = torch.empty(t.shape, dtype=torch.int32)
        codes[:, perm] = qf.unpack_codes(g.codes, 4, K).to(torch.int32)
        tens = qf.gptq_pack(codes, g.sz[..., 0].float(), g.sz[..., 1].float(), 4, 128)
        g_idx = torch.empty(K, dtype=torch.int32)
        g_idx[perm] = (torch.arange(K) // 128).to(torch.int32)
        tens["g_idx"] = g_idx
        for n, v in tens.items():
            qsd[k[:-6] + n] = v
        d = torch.empty_like(t)
        d[:, perm] = qf.dequantize(g)
        deq[k] = d
    w = InMemoryWeights(qsd, dtype=torch.float32)
    w.quant = {"quant_method": "gptq", "bits": 4, "group_size": 128, "zero_offset": 1, "desc_act": True}
    mq = DecoderModel.from_weights(cfg, w, torch.device("cpu"), torch.float32)
    assert all(isinstance(getattr(lw, n), qf.GroupQuantWeight) and getattr(lw, n).perm is not None
               for lw in mq.layers for n in ("qkv_w", "o_w", "gate_up_w", "down_w"))
    md = DecoderModel.from_weights(cfg, InMemoryWeights(deq, dtype=torch.float32), torch.device("cpu"), torch.float32)
    ids = list(range(3, 40))
    a, b = _forward(mq, ids), _forward(md, ids)
    assert torch.allclose(a, b, atol=2e-4), (a - b).abs().max()


@pytest.mark.parametrize("method,tol", [("int4", 0.5), ("eetq", 0.04), ("bitsandbytes-nf4", 0.5), ("hqq-4bit", 0.5)])
def test_model_quantised_on_load_stays_close_to_dense(method, tol):
    cfg = _tiny()
    m = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=6, std=0.05)
    ids = list(range(5, 60))
    want = _forward(m, ids)
    m.quantize(method)
    assert m.quantized == method and isinstance(m.layers[0].qkv_w, qf.GroupQuantWeight)
    got = _forward(m, ids)
    assert ((got - want).norm() / want.norm()).item() < tol


# ------------------------------------------------------------------------------------------------ kernels

@pytest.mark.gpu
@pytest.mark.parametrize("method", ["int4", "eetq", "bitsandbytes-nf4", "bitsandbytes-fp4", "hqq-4bit", "hqq-3bit", "hqq-2bit"])
def test_expansion_kernel_matches_reference(method):
    from lorax_b200.ops import native
    torch.manual_seed(7)
    w = torch.randn(272, 1024) * 0.05
    g = qf.quantize_weight(w, method).to("cuda")
    got = native.wq_dequant(g).float().cpu()
    want = qf.dequantize(g.to("cpu")).to(torch.bfloat16).float()
    assert torch.equal(got, want), (got - want).abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("T", [1, 5, 8, 13, 16, 27, 32])
def test_int4_tensor_core_gemm_matches_fp32_reference(T):
    """out = x . dequant(W)^T straight from the packed codes, against an fp32 product of the same expanded matrix."""
    from lorax_b200.ops import native
    torch.manual_seed(8 + T)
    # one and two row tiles per warp; the last shape (K >= 8192) takes the exact-integer variant at up to 8 tokens
    for N, g, K in ((1040, None, 1536), (1056, None, 1536), (1040, 64, 1536), (1056, 32, 1536), (272, None, 8192), (16384, None, 256)):
        w = torch.randn(N, K) * 0.05
        g = qf.quantize_rtn(w, 4, 128) if g is None else (qf.quantize_hqq(w, 4, g) if g == 64 else qf.quantize_rtn(w, 4, g))
        gd = g.to("cuda")
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        bias = torch.randn(N, device="cuda").to(torch.bfloat16)
        out = torch.full((T, N), 7.0, device="cuda", dtype=torch.bfloat16)
        want = x.float().cpu() @ qf.dequantize(g).t() + bias.float().cpu()
        # general path (scale folded into the operand) and, where the zero points are integers, the exact-integer path
        for flag in ([0, 1] if g.int_zero else [0]):
            out.fill_(7.0)
            rc = native.load().lx_wq4_gemm_ex(x.data_ptr(), x.stride(0), gd.codes.data_ptr(), gd.sz.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                              out.stride(0), T, N, K, gd.group, flag, torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize()
            err = ((out.float().cpu() - want).norm() / want.norm()).item()
            assert err < 6e-3, (T, g.group, flag, err)
        assert g.int_zero == (g.method != "hqq-4bit")


@pytest.mark.gpu
@pytest.mark.parametrize("T", [3, 48])
def test_act_order_gemm_on_gpu_matches_fp32_reference(T):
    """A packed matrix with a column order (act-order GPTQ) through both kernels behind `gemm_wq` (the 4-bit tensor-core GEMM at
    few tokens, expansion + bf16 GEMM above), and through the expansion kernel alone, against fp32 products on the CPU."""
    from lorax_b200.ops import native
    torch.manual_seed(40 + T)
    N, K = 1056, 1536
    w = torch.randn(N, K) * 0.05
    perm = torch.randperm(K)
    g = qf.quantize_rtn(w[:, perm].contiguous(), 4, 128)
    g.perm = perm.to(torch.int32)
    dense = qf.dequantize(g)
    assert ((dense - w).norm() / w.norm()).item() < 0.12          # the order is honoured: it is w, up to 4-bit rounding
    gd = g.to("cuda")
    assert (native.wq_dequant(gd).float().cpu() - dense).abs().max().item() < 2e-3
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    out = native.gemm_wq(x, gd)
    torch.cuda.synchronize()
    want = x.float().cpu() @ dense.t()
    assert ((out.float().cpu() - want).norm() / want.norm()).item() < 6e-3


@pytest.mark.gpu
def test_quantised_gemm_dispatch_and_model_on_gpu():
    from lorax_b200.ops import native
    torch.manual_seed(9)
    N, K = 512, 1024
    w = torch.randn(N, K) * 0.05
    for method in ("int4", "eetq", "bitsandbytes-nf4"):
        g = qf.quantize_weight(w, method)
        gd = g.to("cuda")
        for T in (4, 200):                                  # direct 4-bit kernel / expansion + tcgen05 GEMM
            x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
            got = native.gemm_wq(x, gd)
            want = x.float().cpu() @ qf.dequantize(g).t()
            assert ((got.float().cpu() - want).norm() / want.norm()).item() < 8e-3, (method, T)
    native.workspace(torch.device("cuda")).check_status()
    # a quantised model end to end: GPU kernels against the CPU oracle of the same packed weights
    cfg = _tiny()
    cfg.torch_dtype = "bfloat16"
    cpu = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=6, std=0.05)
    gpu = DecoderModel.random_init(cfg, torch.device("cuda"), torch.bfloat16, seed=6, std=0.05)
    cpu.quantize("int4")
    for lc, lg in zip(cpu.layers, gpu.layers):              # the very same packed matrices on both sides
        for name in ("qkv_w", "o_w", "gate_up_w", "down_w"):
            setattr(lg, name, getattr(lc, name).to("cuda"))
    gpu.quantized = "int4"
    ids = list(range(5, 60))
    a, b = _forward(gpu, ids).float().cpu(), _forward(cpu, ids)
    assert ((a - b).norm() / b.norm()).item() < 0.06


@pytest.mark.parametrize("act_order", [False, True])
def test_gptq_checkpoint_quantiser_writes_a_loadable_checkpoint(tmp_path, act_order):
    """`lorax-server quantize --scheme gptq` (with and without `--act-order`): calibrate, quantise, write the AutoGPTQ layout; the
    result loads packed, and its logits are closer to the dense model's than round-to-nearest at the same bit width."""
    from safetensors.torch import load_file, save_file
    from lorax_b200.server import cli
    from lorax_b200.utils.weights import Weights, weight_files
    cfg = _tiny()
    dense = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=11, std=0.05)
    src, dst = tmp_path / "dense", tmp_path / "gptq"
    src.mkdir()
    save_file(export_hf_state_dict(dense), str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"model_type": "llama", "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                                 "intermediate_size": cfg.intermediate_size, "num_hidden_layers": cfg.num_hidden_layers,
                                                 "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
                                                 "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
                                                 "max_position_embeddings": 2048, "torch_dtype": "float32"}))
    cli.main(["quantize", str(src), str(dst), "--scheme", "gptq", "--nsamples", "8", "--seqlen", "96", "--json-output"] +
             (["--act-order"] if act_order else []))
    out = load_file(str(dst / "model.safetensors"))
    assert "model.layers.0.self_attn.q_proj.qweight" in out and "model.layers.0.self_attn.q_proj.weight" not in out
    assert out["model.layers.1.mlp.down_proj.qweight"].dtype == torch.int32 and "model.embed_tokens.weight" in out
    raw = json.loads((dst / "config.json").read_text())
    assert raw["quantization_config"]["quant_method"] == "gptq" and (dst / "quantize_config.json").exists()
    w = Weights(weight_files(str(dst)), device="cpu", dtype=torch.float32)
    w.quant = checkpoint_quantization(dst, raw)
    mq = DecoderModel.from_weights(cfg, w, torch.device("cpu"), torch.float32)
    assert mq.quantized == "gptq" and isinstance(mq.layers[1].down_w, qf.GroupQuantWeight)
    assert raw["quantization_config"]["desc_act"] is act_order
    if act_order:                # every projection keeps its channel order, and the fused ones share it
        assert all(isinstance(getattr(lw, n), qf.GroupQuantWeight) and getattr(lw, n).perm is not None
                   for lw in mq.layers for n in ("qkv_w", "o_w", "gate_up_w", "down_w"))
        assert not torch.equal(out["model.layers.0.mlp.down_proj.g_idx"].long(), torch.arange(cfg.intermediate_size) // 128)
    else:
        assert mq.layers[0].qkv_w.perm is None
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (64,), generator=g).tolist()
    want = _forward(dense, ids)
    e_gptq = ((_forward(mq, ids) - want).norm() / want.norm()).item()
    dense.quantize("int4")
    e_rtn = ((_forward(dense, ids) - want).norm() / want.norm()).item()
    assert e_gptq < e_rtn, (e_gptq, e_rtn)


def _tiny_mixtral():
    return cfgs.ModelConfig(model_type="mixtral", vocab_size=300, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=1e4, max_position_embeddings=256,
                            num_local_experts=4, num_experts_per_tok=2, torch_dtype="float32")


def test_mixture_of_experts_is_served_packed():
    """Mixtral's experts under weight-only quantisation: one packed matrix per expert, whether quantised on load or read from a
    GPTQ checkpoint, and logits equal to those of the model holding the same matrices expanded."""
    cfg = _tiny_mixtral()
    dense_model = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=9, std=0.05)
    ids = list(range(3, 50))
    # quantised on load
    mq = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=9, std=0.05)
    mq.quantize("int4")
    lw = mq.layers[0]
    assert isinstance(lw.experts_w13, list) and len(lw.experts_w13) == 4 and all(isinstance(t, qf.GroupQuantWeight) for t in lw.experts_w13 + lw.experts_w2)
    md = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=9, std=0.05)
    for a, b in zip(md.layers, mq.layers):
        for n in ("qkv_w", "o_w"):
            setattr(a, n, qf.dequantize(getattr(b, n)))
        a.experts_w13 = torch.stack([qf.dequantize(t) for t in b.experts_w13])
        a.experts_w2 = torch.stack([qf.dequantize(t) for t in b.experts_w2])
    got, want = _forward(mq, ids), _forward(md, ids)
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
    assert not torch.allclose(want, _forward(dense_model, ids), atol=1e-3)      # 4 bits do change the logits
    # read from a GPTQ checkpoint
    sd = export_hf_state_dict(dense_model)
    qsd, deq = {}, {}
    for k, t in sd.items():
        if k.endswith("_proj.weight") or ".experts." in k:
            g = qf.quantize_rtn(t, 4, 128)
            for n, v in qf.gptq_pack(qf.unpack_codes(g.codes, 4, t.shape[1]), g.sz[..., 0].float(), g.sz[..., 1].float(), 4, 128).items():
                qsd[k[:-6] + n] = v
            deq[k] = qf.dequantize(g)
        else:
            qsd[k] = deq[k] = t
    w = InMemoryWeights(qsd, dtype=torch.float32)
    w.quant = {"quant_method": "gptq", "bits": 4, "group_size": 128, "zero_offset": 1}
    mc = DecoderModel.from_weights(cfg, w, torch.device("cpu"), torch.float32)
    assert mc.quantized == "gptq" and isinstance(mc.layers[1].experts_w2, list) and isinstance(mc.layers[1].experts_w2[3], qf.GroupQuantWeight)
    mcd = DecoderModel.from_weights(cfg, InMemoryWeights(deq, dtype=torch.float32), torch.device("cpu"), torch.float32)
    assert isinstance(mcd.layers[1].experts_w2, torch.Tensor)
    a, b = _forward(mc, ids), _forward(mcd, ids)
    assert torch.allclose(a, b, atol=2e-4), (a - b).abs().max()


def test_checkpoint_experts_are_loaded_expert_parallel():
    """A rank of a tensor-parallel group reads only the experts it owns from a checkpoint (rank r of ws: experts
    [r * E / ws, (r + 1) * E / ws)), like a randomly initialised model does."""
    from lorax_b200.parallel.tp import TensorParallel
    cfg = _tiny_mixtral()
    full = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=9, std=0.05)
    sd = export_hf_state_dict(full)
    for rank in (0, 1):
        m = DecoderModel.from_weights(cfg, InMemoryWeights(dict(sd), dtype=torch.float32), torch.device("cpu"), torch.float32,
                                      TensorParallel(rank, 2))
        for lw, fw in zip(m.layers, full.layers):
            assert lw.experts_w13.shape[0] == 2
            assert torch.equal(lw.experts_w13, fw.experts_w13[2 * rank: 2 * rank + 2])
            assert torch.equal(lw.experts_w2, fw.experts_w2[2 * rank: 2 * rank + 2])


@pytest.mark.gpu
def test_quantised_mixture_of_experts_on_gpu():
    """Mixtral with 4-bit experts on the GPU kernels (the direct 4-bit GEMM for a short prompt, expansion + bf16 GEMM for a long
    one) against the CPU oracle holding the very same packed matrices."""
    from lorax_b200.ops import native
    cfg = _tiny_mixtral()
    cfg.torch_dtype = "bfloat16"
    cfg.hidden_size, cfg.head_dim, cfg.intermediate_size = 256, 64, 384
    cpu = DecoderModel.random_init(cfg, torch.device("cpu"), torch.float32, seed=6, std=0.05)
    gpu = DecoderModel.random_init(cfg, torch.device("cuda"), torch.bfloat16, seed=6, std=0.05)
    cpu.quantize("int4")
    for lc, lg in zip(cpu.layers, gpu.layers):
        for name in ("qkv_w", "o_w"):
            setattr(lg, name, getattr(lc, name).to("cuda"))
        lg.experts_w13 = [t.to("cuda") for t in lc.experts_w13]
        lg.experts_w2 = [t.to("cuda") for t in lc.experts_w2]
    gpu.quantized = "int4"
    gpu._native = None
    for n in (20, 90):
        ids = list(range(5, 5 + n))
        a, b = _forward(gpu, ids).float().cpu(), _forward(cpu, ids)
        assert ((a - b).norm() / b.norm()).item() < 0.06, n
    native.workspace(torch.device("cuda")).check_status()
