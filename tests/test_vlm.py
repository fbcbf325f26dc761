"""LLaVA-NeXT: geometry (feature counts, tiling), vision tower + projector + packing against HuggingFace, image rows spliced into
the decoder's prefill, and the shard runtime behind the router with an image in the prompt."""
import base64
import io
import json

import pytest
import torch

from lorax_b200.models import vlm


def _tiny_hf(seed=0):
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaNextConfig, LlavaNextForConditionalGeneration
    torch.manual_seed(seed)
    vc = CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28, patch_size=14,
                          projection_dim=16)
    tc = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False)
    hc = LlavaNextConfig(vision_config=vc, text_config=tc, image_token_index=299, vision_feature_layer=-2,
                         image_grid_pinpoints=[[28, 56], [56, 28], [56, 56], [28, 84], [84, 28]], projector_hidden_act="gelu")
    hc._attn_implementation = "eager"
    hf = LlavaNextForConditionalGeneration(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    return hf, hc


def _tiny_hf_siglip(seed=0):
    """The same model with a SigLIP tower: no class token, biased patch convolution, tanh GELU, strategy "full"."""
    from transformers import LlamaConfig, LlavaNextConfig, LlavaNextForConditionalGeneration, SiglipVisionConfig
    torch.manual_seed(seed)
    vc = SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28, patch_size=14)
    tc = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False)
    hc = LlavaNextConfig(vision_config=vc, text_config=tc, image_token_index=299, vision_feature_layer=-2,
                         vision_feature_select_strategy="full",
                         image_grid_pinpoints=[[28, 56], [56, 28], [56, 56], [28, 84], [84, 28]], projector_hidden_act="gelu")
    hc._attn_implementation = "eager"
    hf = LlavaNextForConditionalGeneration(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    return hf, hc


def _ours(hf, hc):
    from lorax_b200.utils.weights import InMemoryWeights
    cfg = vlm.LlavaNextConfig.from_dict(hc.to_dict())
    cfg.text.torch_dtype = "float32"
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    return vlm.LlavaNextModel.from_weights(cfg, InMemoryWeights(sd, dtype=torch.float32), "cpu", torch.float32)


@pytest.mark.parametrize("size", [(28, 28), (40, 100), (100, 40), (56, 56), (30, 120), (333, 90)])
def test_feature_count_matches_packing(size):
    hf, hc = _tiny_hf()
    m = _ours(hf, hc)
    h, w = size
    bh, bw = vlm.select_best_resolution((h, w), hc.image_grid_pinpoints)
    n_tiles = 1 + (bh // 28) * (bw // 28)
    tiles = torch.randn(n_tiles, 3, 28, 28)
    feats = m.image_features(tiles, (h, w))
    assert feats.shape == (m.num_image_features(h, w), 64)
    with torch.no_grad():
        want = hf.model.get_image_features(pixel_values=tiles[None], image_sizes=torch.tensor([[h, w]]), vision_feature_layer=-2,
                                           vision_feature_select_strategy="default")
    want = want.pooler_output if hasattr(want, "pooler_output") else want
    want = torch.cat(list(want), 0) if isinstance(want, (list, tuple)) else want
    assert want.shape == feats.shape and (want - feats).abs().max().item() < 1e-4


@pytest.mark.parametrize("size", [(28, 28), (40, 100), (333, 90)])
def test_siglip_tower_features_match_hf(size):
    hf, hc = _tiny_hf_siglip()
    m = _ours(hf, hc)
    assert m.config.vision.is_siglip and "cls" not in m.w and m.image_mean == (0.5, 0.5, 0.5)
    h, w = size
    bh, bw = vlm.select_best_resolution((h, w), hc.image_grid_pinpoints)
    tiles = torch.randn(1 + (bh // 28) * (bw // 28), 3, 28, 28)
    feats = m.image_features(tiles, (h, w))
    assert feats.shape == (m.num_image_features(h, w), 64)
    with torch.no_grad():
        want = hf.model.get_image_features(pixel_values=tiles[None], image_sizes=torch.tensor([[h, w]]), vision_feature_layer=-2,
                                           vision_feature_select_strategy="full")
    want = want.pooler_output if hasattr(want, "pooler_output") else want
    want = torch.cat(list(want), 0) if isinstance(want, (list, tuple)) else want
    assert want.shape == feats.shape and (want - feats).abs().max().item() < 1e-4


def test_logits_with_an_image_match_hf():
    from lorax_b200.runtime.kv_cache import KVCache
    from lorax_b200.runtime.runner import ModelRunner, PrefillItem
    hf, hc = _tiny_hf(1)
    m = _ours(hf, hc)
    h, w = 50, 90
    bh, bw = vlm.select_best_resolution((h, w), hc.image_grid_pinpoints)
    tiles = torch.randn(1 + (bh // 28) * (bw // 28), 3, 28, 28)
    n = m.num_image_features(h, w)
    ids = [5, 17, 42] + [299] * n + [7, 9, 200, 31]
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=tiles[None], image_sizes=torch.tensor([[h, w]])).logits[0]
    feats = m.image_features(tiles, (h, w))
    t = m.text
    kv = KVCache(t.config.num_hidden_layers, 16, t.nkv, t.d, t.dtype, t.device)
    r = ModelRunner(t, kv, max_batch=2, max_seq_tokens=256, max_prefill_tokens=256, use_graphs=False)
    got = r.prefill([PrefillItem(ids, 0, [1, 2, 3, 4], all_logprobs=True, embed_index=list(range(3, 3 + n)), embeds=feats)])[2]
    assert (got - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())
    # without the image rows the logits differ: the splice is live
    plain = r.prefill([PrefillItem(ids, 0, [5, 6, 7, 8], all_logprobs=True)])[2]
    assert (plain - want).abs().max().item() > 0.05


def test_pixel_values_match_hf_processor():
    from PIL import Image
    from transformers import LlavaNextImageProcessor
    hf, hc = _tiny_hf()
    m = _ours(hf, hc)
    torch.manual_seed(3)
    proc = LlavaNextImageProcessor(size={"shortest_edge": 28}, crop_size={"height": 28, "width": 28},
                                   image_grid_pinpoints=hc.image_grid_pinpoints)
    for (h, w) in ((40, 100), (100, 37), (28, 28), (61, 59)):
        arr = (torch.rand(h, w, 3) * 255).to(torch.uint8).numpy()
        img = Image.fromarray(arr)
        out = proc(images=img, return_tensors="pt")
        tiles, size = m.pixel_values(img)
        assert size == (h, w) == tuple(out["image_sizes"][0].tolist())
        want = out["pixel_values"][0][: tiles.shape[0]]
        assert want.shape == tiles.shape, (want.shape, tiles.shape)
        assert (want - tiles).abs().max().item() < 0.06, (h, w, (want - tiles).abs().max())


def test_prompt_splitting_and_image_loading():
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", (20, 10), (255, 0, 0)).save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    parts = vlm.split_prompt(f"look ![]({uri}) and ![]({uri})?")
    assert [k for k, _ in parts] == ["text", "image", "text", "image", "text"] and parts[0][1] == "look " and parts[4][1] == "?"
    img = vlm.load_image(parts[1][1])
    assert img.size == (20, 10)
    with pytest.raises(ValueError):
        vlm.load_image("file:///etc/passwd")


@pytest.fixture(scope="module")
def vlm_stack(tmp_path_factory):
    import subprocess
    import time
    import urllib.request
    from tokenizers import Tokenizer, models, pre_tokenizers
    from lorax_b200.csrc import build
    from test_full_stack import ROUTER, _free_port
    build.build_host()
    root = tmp_path_factory.mktemp("vlm")
    hf, hc = _tiny_hf(2)
    mdir = root / "model"
    hf.save_pretrained(str(mdir), safe_serialization=True)
    vocab = {f"w{i}": i for i in range(299)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="w2"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))
    from lorax_b200.config import EngineConfig
    from lorax_b200.server.runtime import VlmRuntime, build_runtime
    from lorax_b200.server.transport import FramedServer
    rt = build_runtime(str(mdir), EngineConfig(max_input_length=96, max_total_tokens=160, max_batch_prefill_tokens=256, compile=False),
                       device="cpu", dtype=torch.float32, source="local", num_blocks=128, max_batch=8)
    assert isinstance(rt, VlmRuntime)
    uds = str(root / "shard")
    srv = FramedServer(rt, uds + "-0.lx").start()
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", uds, "--num-shard", "1",
                             "--max-input-length", "96", "--max-total-tokens", "160", "--max-batch-prefill-tokens", "256",
                             "--model-id", "tiny-llava"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    for _ in range(100):
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                if r.status == 200:
                    break
        except Exception:
            time.sleep(0.1)
    else:
        proc.kill()
        raise RuntimeError("router did not come up: " + proc.stdout.read().decode()[-2000:])
    yield dict(port=port, rt=rt, hf=hf)
    proc.terminate()
    try:
        proc.wait(timeout=10)
    except subprocess.TimeoutExpired:
        proc.kill()
    srv.stop()


def test_image_prompt_through_router_matches_hf(vlm_stack):
    from PIL import Image
    from test_full_stack import _post
    port, rt, hf = vlm_stack["port"], vlm_stack["rt"], vlm_stack["hf"]
    torch.manual_seed(5)
    img = Image.fromarray((torch.rand(40, 70, 3) * 255).to(torch.uint8).numpy())
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    prompt = f"w5 w17 ![]({uri}) w7 w9"
    st, body, _ = _post(port, "/generate", {"inputs": prompt, "parameters": {"max_new_tokens": 6, "details": True}})
    assert st == 200, body
    got = [t["id"] for t in json.loads(body)["details"]["tokens"]]
    # oracle: HuggingFace on the same pixels and the same expanded ids, greedy without a cache
    tiles, size = rt.vlm.pixel_values(img)
    n = rt.vlm.num_image_features(*size)
    ids = [5, 17] + [299] * n + [7, 9]
    assert rt.tokenize(prompt) == ids and json.loads(body)["details"]["prompt_tokens"] == len(ids)
    want = []
    with torch.no_grad():
        for _ in range(6):
            lg = hf(input_ids=torch.tensor([ids + want]), pixel_values=tiles[None], image_sizes=torch.tensor([list(size)])).logits[0, -1]
            want.append(int(lg.argmax()))
    assert got == want
    # text-only prompts take the plain path; two images in one prompt work; a bad image is a client error
    st, body, _ = _post(port, "/generate", {"inputs": "w5 w6 w7", "parameters": {"max_new_tokens": 3}})
    assert st == 200
    st, body, _ = _post(port, "/generate", {"inputs": f"![]({uri}) w3 ![]({uri})", "parameters": {"max_new_tokens": 2}})
    assert st == 200, body
    st, body, _ = _post(port, "/generate", {"inputs": "w1 ![](data:image/png;base64,AAAA) w2", "parameters": {"max_new_tokens": 2}})
    assert st == 422 and json.loads(body)["error_type"] == "validation" and "tokenizer error" in json.loads(body)["error"], body
    assert not rt.seqs
    # the router tokenised these prompts itself: it reads the size of an inline image from its header and computes the feature tokens
    # from the vision configuration the shard handed over; only the broken image was left to the shard
    import urllib.request

    def local_tokenizations():
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5) as r:
            count = [l for l in r.read().decode().splitlines() if l.startswith("lorax_router_tokenizations ")]
        return int(count[0].split()[1])
    before = local_tokenizations()
    assert before >= 3
    # sizes on both sides of the aspect-ratio rules, four encodings: the router's count must be the shard's
    for k, (h, w, fmt) in enumerate([(40, 70, "PNG"), (70, 40, "JPEG"), (33, 33, "GIF"), (20, 97, "BMP"), (97, 21, "WEBP"), (64, 64, "PNG"), (31, 200, "JPEG")]):
        im = Image.fromarray((torch.rand(h, w, 3) * 255).to(torch.uint8).numpy())
        b = io.BytesIO()
        im.save(b, format=fmt)
        u = f"data:image/{fmt.lower()};base64," + base64.b64encode(b.getvalue()).decode()
        p = f"w1 ![]({u}) w2 ![]() w3"
        st, body, _ = _post(port, "/generate", {"inputs": p, "parameters": {"max_new_tokens": 1, "details": True}})
        assert st == 200, (fmt, body)
        assert json.loads(body)["details"]["prompt_tokens"] == len(rt.tokenize(p)), (h, w, fmt)
    assert local_tokenizations() == before + 14          # the two text parts of each of the seven prompts ("![]()" is no image)


def test_router_image_token_count_matches_the_model_over_random_sizes():
    """The router's feature-token count (image size from a PNG header, any-resolution formula) against the model's own over 2000 random
    sizes; references it cannot size are left to the shard."""
    import random
    import struct
    import zlib
    from lorax_b200.models.vlm import select_best_resolution, unpadded_grid
    from lorax_b200.router.native import image_token_count
    pol = {"kind": "llava_next", "image_token": 9, "image_size": 336, "patch_size": 14, "extra_tokens": 1, "strategy": "default",
           "pinpoints": [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]]}

    def png_header(w, h):
        ihdr = struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)
        return b"\x89PNG\r\n\x1a\n" + struct.pack(">I", 13) + b"IHDR" + ihdr + struct.pack(">I", zlib.crc32(b"IHDR" + ihdr))
    rng = random.Random(0)
    side = 336 // 14
    for _ in range(2000):
        h, w = rng.randint(1, 3000), rng.randint(1, 3000)
        bh, bw = select_best_resolution((h, w), pol["pinpoints"])
        _, rows, _, cols = unpadded_grid((h, w), (bh // 336 * side, bw // 336 * side))
        want = side * side + rows * (cols + 1)
        assert image_token_count(pol, "data:image/png;base64," + base64.b64encode(png_header(w, h)).decode()) == want, (h, w)
    assert image_token_count({"kind": "one_per_image", "image_token": 3}, "data:image/png;base64," + base64.b64encode(png_header(5, 5)).decode()) == 1
    for uri in ("https://example.com/a.png", "data:image/png;base64,AAAA", "data:text/plain,hello", "data:image/tiff;base64," + base64.b64encode(b"II*\0" * 8).decode()):
        assert image_token_count(pol, uri) == -1
    assert image_token_count({}, "data:image/png;base64," + base64.b64encode(png_header(5, 5)).decode()) == -1


def test_router_cuts_prompts_at_image_references_like_the_shard():
    import random
    from lorax_b200.models.vlm import split_prompt
    from lorax_b200.router.native import split_image_prompt
    rng = random.Random(4)
    pieces = ["![](", ")", "![]", "(", "a", " b ", "data:x", "![]()", "!", "[", "]", "é", "\n"]
    for _ in range(3000):
        text = "".join(rng.choice(pieces) for _ in range(rng.randint(0, 12)))
        assert split_image_prompt(text) == split_prompt(text), repr(text)
