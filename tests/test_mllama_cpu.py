"""Mllama (Llama 3.2 Vision) against the Hugging Face implementation on a tiny random model: image geometry, vision tower,
cross-attention masks, prompt logits with and without images, and greedy decoding through the per-request state."""

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import MllamaConfig as HFConfig, MllamaForConditionalGeneration  # noqa: E402
from transformers.models.mllama.image_processing_mllama import get_image_size_fit_to_canvas, get_optimal_tiled_canvas  # noqa: E402

from lorax_b200.models import mllama as M  # noqa: E402
from lorax_b200.utils.weights import InMemoryWeights as DictWeights  # noqa: E402

IMG = 40          # image token id (vocab_size)


@pytest.fixture(scope="module")
def pair():
    torch.manual_seed(0)
    cfg = HFConfig(
        vision_config=dict(hidden_size=32, num_hidden_layers=4, num_global_layers=2, attention_heads=4, intermediate_size=64,
                           vision_output_dim=32 * 3, image_size=28, patch_size=14, max_num_tiles=4, intermediate_layers_indices=[1, 3]),
        text_config=dict(vocab_size=IMG, hidden_size=48, num_hidden_layers=5, num_attention_heads=4, num_key_value_heads=2,
                         intermediate_size=96, cross_attention_layers=[1, 3], max_position_embeddings=256, eos_token_id=1,
                         pad_token_id=0, rope_parameters={"rope_type": "default", "rope_theta": 10000.0}),
        image_token_index=IMG)
    hf = MllamaForConditionalGeneration(cfg).to(torch.float32).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():          # gates start at zero: make every branch count
            if "gate" in n and p.numel() == 1:
                p.fill_(0.7)
    ours_cfg = M.MllamaConfig.from_dict(cfg.to_dict())
    ours = M.MllamaModel.from_weights(ours_cfg, DictWeights({k: v.detach() for k, v in hf.state_dict().items()}), "cpu", torch.float32)
    return hf, ours, cfg


def test_image_geometry_matches_the_processor():
    for h, w in [(20, 90), (300, 40), (57, 57), (28, 28), (100, 130), (5, 5), (400, 60)]:
        ch, cw = M.optimal_canvas(h, w, 4, 28)
        assert (ch, cw) == tuple(int(x) for x in get_optimal_tiled_canvas(h, w, 4, 28))
        assert M.fit_to_canvas(h, w, ch, cw, 28) == tuple(int(x) for x in get_image_size_fit_to_canvas(h, w, ch, cw, 28))


def test_cross_attention_spans():
    I = IMG
    assert M.cross_attention_spans([3, 4, 5], I) == []
    assert M.cross_attention_spans([3, I, 5, 6], I) == [(1, -1)]
    assert M.cross_attention_spans([I, 5, I, 6, 7], I) == [(0, 2), (2, -1)]
    assert M.cross_attention_spans([I, I, 6, 7], I) == [(0, -1), (1, -1)]          # consecutive images reach equally far


def _image(h, w, seed):
    from PIL import Image
    rng = np.random.default_rng(seed)
    return Image.fromarray(rng.integers(0, 256, (h, w, 3), dtype=np.uint8))


def _hf_inputs(ours, ids, images):
    """pixel_values / aspect ratio tensors / dense cross-attention mask in the layout the HF model expects (batch of one)."""
    v = ours.config.vision
    tiles = torch.stack([im[0] for im in images])[None]                                   # [1, images, tiles, 3, S, S]
    ar_ids = torch.tensor([[im[1] for im in images]])
    ar_mask = torch.zeros(1, len(images), v.max_num_tiles, dtype=torch.long)
    for i, im in enumerate(images):
        ar_mask[0, i, : im[2]] = 1
    cam = torch.zeros(1, len(ids), len(images), v.max_num_tiles, dtype=torch.long)
    for i, ((a, b), im) in enumerate(zip(M.cross_attention_spans(ids, IMG), images)):
        cam[0, a:(len(ids) if b < 0 else b), i, : im[2]] = 1
    return dict(pixel_values=tiles, aspect_ratio_ids=ar_ids, aspect_ratio_mask=ar_mask, cross_attention_mask=cam)


def test_vision_tower_matches_hf(pair):
    hf, ours, cfg = pair
    for h, w in [(30, 70), (60, 25)]:
        tiles, ar, nt = ours.pixel_values(_image(h, w, h))
        got = ours.vision_features(tiles, ar, nt)
        mask = torch.zeros(1, 1, 4, dtype=torch.long)
        mask[0, 0, :nt] = 1
        with torch.no_grad():
            want = hf.model.vision_model(pixel_values=tiles[None, None], aspect_ratio_ids=torch.tensor([[ar]]), aspect_ratio_mask=mask).last_hidden_state
            want = hf.model.multi_modal_projector(want).reshape(-1, cfg.text_config.hidden_size)
        live = nt * ours.config.vision.num_patches
        assert torch.allclose(got[:live], want[:live], atol=2e-4, rtol=1e-3)


@pytest.mark.parametrize("ids,sizes", [([2, IMG, 5, 9, 11, 3, 7], [(30, 70)]),                 # text in front of the image: a masked-out row
                                       ([IMG, 5, 9, IMG, 11, 3, 7, 8], [(28, 28), (60, 25)]),    # two images, each read by its own span
                                       ([2, 5, 9, 11], [])])                                    # no image: cross-attention layers skipped
def test_prompt_logits_and_greedy_decoding_match_hf(pair, ids, sizes):
    hf, ours, cfg = pair
    images = [ours.pixel_values(_image(h, w, 7 + i)) for i, (h, w) in enumerate(sizes)]
    st = ours.encode(ids, images)
    with torch.no_grad():
        got = [ours.decode_step([st])[0]]
        kw = _hf_inputs(ours, ids, images) if images else {}
        out = hf(input_ids=torch.tensor([ids]), use_cache=True, **kw)
        want = [out.logits[0, -1]]
        assert torch.allclose(got[0], want[0], atol=3e-4, rtol=1e-3)
        # three more tokens through both caches
        past = out.past_key_values
        for _ in range(3):
            tok = int(want[-1].argmax())
            assert int(got[-1].argmax()) == tok
            st.last_token = tok
            got.append(ours.decode_step([st])[0])
            step_kw = {}
            if images:
                ids = ids + [tok]
                cam = _hf_inputs(ours, ids, images)["cross_attention_mask"]
                cam[0, -1] = cam[0, -2]                    # generated tokens read what the last prompt token read
                step_kw["cross_attention_mask"] = cam
            out = hf(input_ids=torch.tensor([[tok]]), past_key_values=past, use_cache=True, **step_kw)
            past = out.past_key_values
            want.append(out.logits[0, -1])
            assert torch.allclose(got[-1], want[-1], atol=3e-4, rtol=1e-3)


def test_mllama_runtime_serves_prompts_with_images(pair, tmp_path):
    """`build_runtime` on an mllama checkpoint gives the per-request runtime: markdown image links become `<|image|>` tokens, the
    image is fetched and tiled once, and Prefill + Decode produce the tokens the model produces when driven directly."""
    import base64
    import io
    from tokenizers import Tokenizer, models, pre_tokenizers
    from lorax_b200.config import EngineConfig
    from lorax_b200.server.runtime import MllamaRuntime, build_runtime
    hf, ours, cfg = pair
    mdir = tmp_path / "model"
    hf.save_pretrained(str(mdir), safe_serialization=True)
    tok = Tokenizer(models.WordLevel({f"w{i}": i for i in range(IMG)}, unk_token="w2"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))
    rt = build_runtime(str(mdir), EngineConfig(max_input_length=64, max_total_tokens=96, compile=False), device="cpu", dtype=torch.float32,
                       source="local")
    assert isinstance(rt, MllamaRuntime)
    buf = io.BytesIO()
    _image(30, 70, 3).save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    text = f"w5 ![]({uri}) w9 w11 w3"
    ids = rt.tokenize(text, add_special=False)
    assert ids == [5, IMG, 9, 11, 3]
    pb = rt.pb
    req = pb.Request(id=7, inputs=text, truncate=64,
                     parameters=pb.NextTokenChooserParameters(temperature=1.0, top_p=1.0, typical_p=1.0, repetition_penalty=1.0),
                     stopping_parameters=pb.StoppingCriteriaParameters(max_new_tokens=4, ignore_eos_token=True))
    resp = rt.prefill(pb.PrefillRequest(batch=pb.Batch(id=1, requests=[req], size=1, max_tokens=96)))
    got = list(resp.generations[0].next_tokens.ids)
    batch = resp.batch
    while len(got) < 4:
        resp = rt.decode(pb.DecodeRequest(batches=[batch]))
        got += list(resp.generations[0].next_tokens.ids)
        if resp.HasField("batch"):
            batch = resp.batch
    # the same prompt driven directly
    from lorax_b200.models.vlm import load_image
    st = rt.model.encode(ids, [rt.model.pixel_values(load_image(uri))])
    want = []
    with torch.no_grad():
        for _ in range(4):
            tokn = int(rt.model.decode_step([st])[0].argmax())
            want.append(tokn)
            st.last_token = tokn
    assert got == want
    assert not rt.seqs and not rt.states                  # finished requests leave nothing behind
