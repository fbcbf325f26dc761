"""The router's C++ tokenizer against the HuggingFace `tokenizers` library: same ids for every pipeline the router implements
(byte-level BPE with the GPT-2 and the Llama-3 split patterns, SentencePiece-style BPE with byte fallback, WordPiece with the
BERT normaliser, Unigram, WordLevel), special tokens inside the text, Unicode normalisation forms, and the fallback signal for
files it does not implement.  The reference router tokenises with that library (router/src/validation.rs:44-118)."""

import json
import random
import unicodedata

import pytest

tokenizers = pytest.importorskip("tokenizers")
from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, processors, trainers  # noqa: E402

from lorax_b200.router.native import RouterTokenizer, regex_find_all, unicode_normalize  # noqa: E402

WORDS = ("the quick brown fox jumps over lazy dog tokenizer adapter LoRA B200 serving request batch prefill decode "
         "naïve café résumé straße Ελληνικά привет мир 日本語 中文 字 한국어 emoji 🙂 🚀 don't we're I'll it's 12345 3.14 "
         "x=y+z; foo_bar(baz) <html> &amp; tab\there new\nline  double  space trailing ").split(" ")


def corpus(n=400, seed=0):
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        k = rng.randint(1, 24)
        out.append(" ".join(rng.choice(WORDS) for _ in range(k)))
    return out


SAMPLES = corpus(120, seed=7) + [
    "", " ", "  leading and trailing  ", "Hello, world!", "don't stop: we're here; I'll go. IT'S FINE", "a\n\nb\r\nc\t\td   ",
    "price: $1,234.56 (approx.) 100% sure", "naïve café — “quoted” … ½ ① ﬁn", "日本語のテキストと中文字符 mixed with English",
    "한국어 텍스트 각", "🙂🚀 emoji‍ sequence 👩‍👩‍👧", "é vs é and ẛ̣ क़", "tabs\tand\x00nul\x7f",
    "x" * 300, "unknownwordzzzqqq " * 5, "İstanbul ΣΊΣΥΦΟΣ ǅ", "ctl\x01\x08\x0b\x1f\x7f\x8f\x9f sp\x0c\u1680\u200b\u200f\u2028\u2581\ufeff\ufffd end",
]


def check(tmp_path, tok: Tokenizer, samples=SAMPLES, special=(True, False)):
    path = tmp_path / "tokenizer.json"
    tok.save(str(path))
    mine = RouterTokenizer(str(path), workers=2)
    for text in samples:
        for add in special:
            try:
                want = tok.encode(text, add_special_tokens=add).ids
            except Exception:
                with pytest.raises(ValueError):
                    mine.encode(text, add)
                continue
            got = mine.encode(text, add)
            assert got == want, (text, add, got[:40], want[:40])
    mine.close()


GPT2_SPLIT = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
LLAMA3_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
QWEN2_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")


def byte_level_bpe(pre, normalizer=None, special=("<|begin_of_text|>", "<|eot_id|>"), ignore_merges=False):
    tok = Tokenizer(models.BPE(ignore_merges=ignore_merges))
    if normalizer is not None:
        tok.normalizer = normalizer
    tok.pre_tokenizer = pre
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=list(special), initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(corpus(), trainer)
    return tok


def test_gpt2_style_byte_level_bpe(tmp_path):
    tok = byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True))
    check(tmp_path, tok)
    tok2 = byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=True, use_regex=True))
    check(tmp_path, tok2)


def test_llama3_style_split_pattern_template_and_special_tokens_in_text(tmp_path):
    pre = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(LLAMA3_SPLIT), behavior="isolated", invert=False),
                                   pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok = byte_level_bpe(pre, ignore_merges=True)
    bos = tok.token_to_id("<|begin_of_text|>")
    tok.post_processor = processors.Sequence([
        processors.ByteLevel(trim_offsets=False),
        processors.TemplateProcessing(single="<|begin_of_text|> $A", special_tokens=[("<|begin_of_text|>", bos)])])
    extra = ["<|begin_of_text|>system prompt<|eot_id|>user says hi<|eot_id|>", "text<|eot_id|> <|eot_id|>more", "<|eot_id", "1234567 12 1 0000"]
    check(tmp_path, tok, SAMPLES + extra)


def test_qwen2_style_nfc_normaliser_and_single_digits(tmp_path):
    pre = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(QWEN2_SPLIT), behavior="isolated", invert=False),
                                   pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok = byte_level_bpe(pre, normalizer=normalizers.NFC(), special=("<|endoftext|>", "<|im_start|>", "<|im_end|>"))
    check(tmp_path, tok, SAMPLES + ["<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n"])


def sentencepiece_bpe(legacy: bool):
    tok = Tokenizer(models.BPE(unk_token="<unk>", fuse_unk=True, byte_fallback=True))
    special = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    if legacy:           # Llama-2 / Mistral: the normaliser writes the metaspace, no pre-tokenizer
        tok.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    else:
        tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="first", split=False)
    trainer = trainers.BpeTrainer(vocab_size=700, special_tokens=special, show_progress=False)
    # train on metaspace-split words so merges do not cross words much, as SentencePiece does
    trainee = Tokenizer(models.BPE(unk_token="<unk>", fuse_unk=True, byte_fallback=True))
    trainee.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="always", split=True)
    trainee.train_from_iterator(corpus(), trainer)
    state = json.loads(trainee.to_str())
    mine = json.loads(tok.to_str())
    mine["model"] = state["model"]
    mine["added_tokens"] = [a for a in state["added_tokens"] if a["content"] in ("<unk>", "<s>", "</s>")]
    tok = Tokenizer.from_str(json.dumps(mine))
    tok.post_processor = processors.TemplateProcessing(single="<s> $A", special_tokens=[("<s>", tok.token_to_id("<s>"))])
    return tok


@pytest.mark.parametrize("legacy", [True, False])
def test_sentencepiece_style_bpe_with_byte_fallback(tmp_path, legacy):
    tok = sentencepiece_bpe(legacy)
    check(tmp_path, tok, SAMPLES + ["</s> after eos", "mid<s>dle", "<s>", "▁already▁meta"])


def test_bert_wordpiece(tmp_path):
    tok = Tokenizer(models.WordPiece(unk_token="[UNK]"))
    tok.normalizer = normalizers.BertNormalizer(lowercase=True)
    tok.pre_tokenizer = pre_tokenizers.BertPreTokenizer()
    trainer = trainers.WordPieceTrainer(vocab_size=500, special_tokens=["[UNK]", "[CLS]", "[SEP]", "[PAD]", "[MASK]"], show_progress=False)
    tok.train_from_iterator(corpus(), trainer)
    tok.post_processor = processors.BertProcessing(("[SEP]", tok.token_to_id("[SEP]")), ("[CLS]", tok.token_to_id("[CLS]")))
    check(tmp_path, tok, SAMPLES + ["a [MASK] token", "[CLS] inside [SEP]"])
    cased = Tokenizer.from_str(tok.to_str())
    cased.normalizer = normalizers.BertNormalizer(lowercase=False, strip_accents=False)
    check(tmp_path, cased)


def test_unigram_with_metaspace(tmp_path):
    tok = Tokenizer(models.Unigram())
    tok.normalizer = normalizers.Sequence([normalizers.NFKC(), normalizers.Replace(Regex(" {2,}"), " ")])
    tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="always")
    trainer = trainers.UnigramTrainer(vocab_size=400, special_tokens=["<pad>", "</s>", "<unk>"], unk_token="<unk>", show_progress=False)
    tok.train_from_iterator(corpus(), trainer)
    tok.post_processor = processors.TemplateProcessing(single="$A </s>", special_tokens=[("</s>", tok.token_to_id("</s>"))])
    check(tmp_path, tok)


def test_word_level_whitespace_digits_and_punctuation(tmp_path):
    vocab = {w: i for i, w in enumerate(dict.fromkeys(["<unk>"] + [w.lower() for w in WORDS] + list("0123456789.,;!?()=+")))}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.normalizer = normalizers.Sequence([normalizers.Nmt(), normalizers.NFD(), normalizers.StripAccents(), normalizers.Lowercase(), normalizers.Strip()])
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Whitespace(), pre_tokenizers.Digits(individual_digits=True), pre_tokenizers.Punctuation()])
    check(tmp_path, tok)
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.WhitespaceSplit(), pre_tokenizers.Digits(individual_digits=False)])
    check(tmp_path, tok)
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.CharDelimiterSplit(" "), pre_tokenizers.Punctuation("merged_with_previous")])
    check(tmp_path, tok)
    no_unk = Tokenizer(models.WordLevel(vocab))                 # a word outside the vocabulary is an error, here as there
    no_unk.pre_tokenizer = pre_tokenizers.Whitespace()
    check(tmp_path, no_unk, ["the quick fox", "the zzzz fox"])


def test_added_tokens_with_strip_single_word_and_normalised_content(tmp_path):
    tok = byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True), normalizer=normalizers.Lowercase(), special=("<s>",))
    tok.add_special_tokens([tokenizers.AddedToken("<mask>", lstrip=True, rstrip=False), tokenizers.AddedToken("<sep>", rstrip=True)])
    tok.add_tokens([tokenizers.AddedToken("WordTok", single_word=True, normalized=True), tokenizers.AddedToken("RawTok", normalized=False),
                    tokenizers.AddedToken("<s>long", normalized=False)])
    samples = ["a   <mask>   b", "x<sep>   y <sep>", "WordTok wordtok aWordTok WordTokb (wordtok)", "RawTok rawtok RAWTOK", "<s>long<s>lo <s>",
               "<mask><mask> <sep><s>"]
    check(tmp_path, tok, SAMPLES[:30] + samples)


def test_unicode_normalisation_forms_match_unicodedata():
    rng = random.Random(3)
    pool = [chr(c) for c in list(range(0x20, 0x250)) + list(range(0x300, 0x370)) + list(range(0x1E00, 0x2000)) + list(range(0x3040, 0x3100))
            + list(range(0xAC00, 0xAC40)) + list(range(0x1100, 0x1120)) + list(range(0x1161, 0x1176)) + list(range(0x11A8, 0x11C3))
            + list(range(0xFB00, 0xFB07)) + list(range(0xFF00, 0xFF60)) + [0x0958, 0x0F73, 0x1D15E, 0x2126, 0x212B, 0x1F600]]
    for _ in range(300):
        s = "".join(rng.choice(pool) for _ in range(rng.randint(1, 12)))
        for form in ("NFC", "NFD", "NFKC", "NFKD"):
            assert unicode_normalize(s, form) == unicodedata.normalize(form, s), (form, [hex(ord(c)) for c in s])
    assert unicode_normalize("İSTANBUL ΣΊΣ Straße", "lower") == "".join(c.lower() for c in "İSTANBUL ΣΊΣ Straße")


def test_unsupported_files_are_refused_with_the_reason(tmp_path):
    tok = byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True))
    state = json.loads(tok.to_str())
    state["normalizer"] = {"type": "Precompiled", "precompiled_charsmap": "AAAA"}
    p = tmp_path / "a.json"
    p.write_text(json.dumps(state))
    with pytest.raises(ValueError, match="Precompiled"):
        RouterTokenizer(str(p))
    state["normalizer"] = None
    state["pre_tokenizer"] = {"type": "Split", "pattern": {"Regex": r"(?P<x>a)\1|(?<=a+)b"}, "behavior": "Isolated", "invert": False}
    p.write_text(json.dumps(state))
    with pytest.raises(ValueError, match="regex"):
        RouterTokenizer(str(p))
    with pytest.raises(ValueError, match="cannot read"):
        RouterTokenizer(str(tmp_path / "missing.json"))


def test_pool_serves_concurrent_callers(tmp_path):
    import threading
    tok = byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True))
    path = tmp_path / "tokenizer.json"
    tok.save(str(path))
    mine = RouterTokenizer(str(path), workers=3)
    texts = corpus(64, seed=11)
    want = [tok.encode(t).ids for t in texts]
    got = [None] * len(texts)

    def work(lo):
        for i in range(lo, len(texts), 8):
            got[i] = mine.encode(texts[i])
    threads = [threading.Thread(target=work, args=(k,)) for k in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert got == want


def test_llama_tokenizer_class_gets_the_bos_template_on_both_sides(tmp_path):
    """A Llama tokenizer file carries no post-processor; transformers adds BOS (and EOS when configured) at load time and the
    reference router does the same for tokenizer classes LlamaTokenizer / LlamaTokenizerFast (router/src/main.rs:587-655).  The
    shard applies the override when it loads the file, and the router tokenises from the shard's copy."""
    from lorax_b200.server.runtime import load_tokenizer
    tok = sentencepiece_bpe(legacy=True)
    state = json.loads(tok.to_str())
    state["post_processor"] = None
    mdir = tmp_path / "m"
    mdir.mkdir()
    (mdir / "tokenizer.json").write_text(json.dumps(state))
    (mdir / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "LlamaTokenizerFast", "bos_token": {"content": "<s>"},
                                                            "eos_token": "</s>", "add_eos_token": True}))
    loaded = load_tokenizer(str(mdir))
    bos, eos = loaded.token_to_id("<s>"), loaded.token_to_id("</s>")
    ids = loaded.encode("hello world").ids
    assert ids[0] == bos and ids[-1] == eos and loaded.encode("hello world", add_special_tokens=False).ids == ids[1:-1]
    (tmp_path / "served.json").write_text(loaded.to_str())
    mine = RouterTokenizer(str(tmp_path / "served.json"))
    assert mine.encode("hello world") == ids
    (mdir / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "GPT2Tokenizer", "bos_token": "<s>"}))
    assert load_tokenizer(str(mdir)).encode("hello world").ids == ids[1:-1]
    # padding and truncation saved with the file are dropped on load: both sides see the whole text and nothing else
    state["padding"] = {"strategy": {"Fixed": 16}, "direction": "Right", "pad_to_multiple_of": None, "pad_id": 0, "pad_type_id": 0, "pad_token": "<unk>"}
    state["truncation"] = {"direction": "Right", "max_length": 4, "strategy": "LongestFirst", "stride": 0}
    (mdir / "tokenizer.json").write_text(json.dumps(state))
    assert Tokenizer.from_file(str(mdir / "tokenizer.json")).encode("hello world").ids != ids[1:-1]
    assert load_tokenizer(str(mdir)).encode("hello world").ids == ids[1:-1]


@pytest.mark.parametrize("behavior", ["isolated", "removed", "merged_with_previous", "merged_with_next", "contiguous"])
def test_zero_width_and_look_behind_split_patterns(tmp_path, behavior):
    """Look-behind, word boundaries and zero-width matches (camelCase cuts) in a Split pattern, under every split behaviour."""
    pattern = r"(?<=[a-z])(?=[A-Z])|\b\d+\b|(?<!\S)-"
    pre = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pattern), behavior=behavior, invert=False),
                                   pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok = byte_level_bpe(pre)
    extra = ["camelCaseWordsHere and snake_case 123 a1b2 -dash non-dash", "fooBar", "XMLHttpRequest 42", "- -a b-", "aB", "a", "9"]
    check(tmp_path, tok, SAMPLES[:40] + extra)


def precompiled_unigram():
    """A T5 / XLM-R style tokenizer: Unigram behind SentencePiece's compiled nmt_nfkc character map, taken from a model trained here."""
    spm = pytest.importorskip("sentencepiece")
    from sentencepiece import sentencepiece_model_pb2 as pb
    import io
    import os
    model = io.BytesIO()
    devnull = os.open(os.devnull, os.O_WRONLY)
    saved = os.dup(2)
    os.dup2(devnull, 2)                      # the trainer logs to stderr
    try:
        spm.SentencePieceTrainer.train(sentence_iterator=iter(corpus(600, seed=2)), model_writer=model, vocab_size=300, model_type="unigram",
                                       hard_vocab_limit=False)
    finally:
        os.dup2(saved, 2)
        os.close(devnull)
        os.close(saved)
    proto = pb.ModelProto()
    proto.ParseFromString(model.getvalue())
    charsmap = proto.normalizer_spec.precompiled_charsmap
    assert len(charsmap) > 100_000
    vocab = [(p.piece, p.score) for p in proto.pieces]
    tok = Tokenizer(models.Unigram(vocab, unk_id=0))
    tok.normalizer = normalizers.Sequence([normalizers.Precompiled(charsmap), normalizers.Replace(Regex(" {2,}"), " ")])
    tok.pre_tokenizer = pre_tokenizers.Metaspace(replacement="▁", prepend_scheme="always")
    tok.post_processor = processors.TemplateProcessing(single="$A </s>", special_tokens=[("</s>", 2)])
    return tok


HARD_UNICODE = ["ﬁn ① ½ Ⅷ ｆｕｌｌ　ｗｉｄｔｈ ㎏ ℃ Å", "é ạ̈ ố ́alone", "اَّلسَّلَامُ عَلَيْكُمْ ؀123", "한국어 각 한́",
                "a\r\nb\rc\nd\t\te", "👩‍👩‍👧 ❤‍🔥 🇩🇪🇫🇷 👍🏽", "क्षत्रिय हिन्दी กำลัง น้ำ", "soft­hyphen zero​width ‍j ﻿bom", "ǅ ﬃ ẛ̣ ™ ² ³ ¼ № ㍿",
                "x́́́́ ำ ःa", "", " ", "   multiple   spaces   "]


def test_sentencepiece_precompiled_character_map(tmp_path):
    """SentencePiece's compiled character map applied grapheme cluster by grapheme cluster, in front of a Unigram model."""
    tok = precompiled_unigram()
    check(tmp_path, tok, SAMPLES + HARD_UNICODE)


def test_byte_level_normaliser_and_fixed_length_chunks(tmp_path):
    """The byte-level alphabet applied by the normaliser (newer tokenizer files) with a plain split pattern behind it, and the
    FixedLength pre-tokenizer."""
    tok = Tokenizer(models.BPE())
    tok.normalizer = normalizers.ByteLevel()
    tok.pre_tokenizer = pre_tokenizers.Split(Regex("Ġ?[^Ġ]+"), behavior="isolated")
    trainer = trainers.BpeTrainer(vocab_size=500, special_tokens=["<|endoftext|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(corpus(), trainer)
    check(tmp_path, tok, SAMPLES + ["a<|endoftext|>b"])
    tok.pre_tokenizer = pre_tokenizers.FixedLength(3)
    check(tmp_path, tok, SAMPLES[:40])
    tok.pre_tokenizer = pre_tokenizers.UnicodeScripts()           # cuts where the script changes
    check(tmp_path, tok, SAMPLES + ["Apples are りんご 林檎", " a  b ", "   ", "abc123, def! привет мир ーー カタカナ"])


REGEX_CASES = [
    GPT2_SPLIT, LLAMA3_SPLIT, QWEN2_SPLIT, r"\w+|[^\w\s]+", r" {2,}", r"a+?b", r"(a|ab)(c|bcd)(d*)", r"x*", r"(?i)straße|ǅ", r"[A-Z][a-z]+|[A-Z]+(?![a-z])",
    r"\d{2,4}-\d{1,2}", r"(?<=\s)\S+|^\S+", r"(?<![a-z])[a-z]{3}\b", r"\p{Lu}\p{Ll}*|\p{Nd}+|\p{P}", r"[^\x00-\x7f]+", r"[\u4e00-\u9fff]|[a-z]+",
    r"\p{Han}+|\p{Hiragana}+|\p{IsKatakana}+|\p{Script=Latin}+|\p{sc=Cyrillic}+|\P{Common}", r"(?:ab)+c?|b{2,}?", r"\S+\s*?", r".+?(?=,|$)", r"[\-\]\[]+", r"\bfoo\B|\Bbar\b", r"(?i:[a-c]+)x", r"'(?:[sdmt]|ll|ve|re)",
]
REGEX_TEXTS = ["Hello, World! it's 2024-05-17 and we're HERE: fooBar barfoo food", "  leading  spaces\tand\nnewlines\r\n  ", "STRASSE straße Ǆ ǅ ǆ",
               "日本語のテキスト abc 中文 XYZabc ABCx aBcX привет ーー",  "aab abcd abbbcdd xx-][-", "", "a", "1234-5 12-345 123456-78", "naïve café — “q” … ½ ①"]


@pytest.mark.parametrize("pattern", REGEX_CASES)
def test_regex_engine_matches_like_a_backtracking_reference(pattern):
    """The router's regex engine against the `regex` package (same leftmost, first-alternative-wins semantics as the engine the
    library splits with) on the split patterns of well-known tokenizers and on constructs each alone."""
    rx = pytest.importorskip("regex")
    flags = rx.V0
    want_re = rx.compile(pattern, flags)
    for text in REGEX_TEXTS:
        want = [[m.start(), m.end()] for m in want_re.finditer(text)]
        assert regex_find_all(pattern, text) == want, (pattern, text)


def test_regex_engine_refuses_what_it_does_not_implement():
    for pattern in [r"(a)\1", r"(?P<n>a)", r"(?<=a+)b", r"[[:alpha:]]", r"a{1000}"]:
        with pytest.raises(ValueError):
            regex_find_all(pattern, "aab")


def test_bpe_with_word_suffix_and_continuation_prefix(tmp_path):
    """Older BPE files: `</w>` closes a word (CLIP, GPT-1), `##` marks a continuation."""
    for kw in ({"end_of_word_suffix": "</w>"}, {"continuing_subword_prefix": "##"}, {"continuing_subword_prefix": "@@", "end_of_word_suffix": "</w>"}):
        tok = Tokenizer(models.BPE(unk_token="<unk>", **kw))
        tok.normalizer = normalizers.Sequence([normalizers.NFC(), normalizers.Lowercase()])
        tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Whitespace(), pre_tokenizers.Digits(individual_digits=True)])
        trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<unk>", "<|startoftext|>", "<|endoftext|>"], show_progress=False, **kw)
        tok.train_from_iterator(corpus(), trainer)
        check(tmp_path, tok)


def test_random_strings_of_awkward_characters(tmp_path):
    """Seeded fuzz: control characters, combining marks, joiners, regional indicators, Hangul jamo, private-use and replacement
    characters and pieces of special tokens, against the library, for a byte-level and a SentencePiece-style tokenizer."""
    rng = random.Random(1)
    alphabet = [chr(c) for c in list(range(0, 0x250)) + [0x300, 0x301, 0x200D, 0x1F600, 0x1F1E6, 0xAC00, 0x1100, 0x1161, 0x11A8, 0xFE0F, 0x0600, 0x0E33,
                                                          0xFFFD, 0x2028, 0x3000, 0x4E2D, 0xE000]] + ["<s>", "</s>", "<|eot_id|>", "<|begin_of_text|>"]
    strings = ["".join(rng.choice(alphabet) for _ in range(rng.randint(0, 40))) for _ in range(600)]
    check(tmp_path, byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)), strings, special=(True,))
    check(tmp_path, sentencepiece_bpe(True), strings, special=(True,))
