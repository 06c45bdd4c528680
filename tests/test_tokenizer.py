"""Native BPE tokenizer against the Hugging Face `tokenizers` implementation on a freshly trained vocabulary."""
import os

import pytest


def _train(tmp_path):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer as HFT, decoders, models, pre_tokenizers, trainers
    pat = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
           r"|\s+(?!\S)|\s+")
    tok = HFT(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(pat), behavior="isolated"),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    corpus = ["Hello world! It's 2024, and we're testing   tokenizers.\n\nNew paragraph: foo_bar(baz) = 3.14159;",
              "def f(x):\n    return x**2  # comment\n", "Ünïcödé tëxt — 日本語のテキスト 12345 и русский",
              "  leading spaces and\ttabs\r\nwindows line"] * 50
    tr = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                             initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(corpus, tr)
    tok.save(os.path.join(tmp_path, "tokenizer.json"))
    return tok, corpus


def test_bpe_matches_hf_and_roundtrips(tmp_path):
    from volta_engine_b200.loader.tokenizer import Tokenizer
    hf, corpus = _train(str(tmp_path))
    t = Tokenizer.load(str(tmp_path))
    cases = corpus[:4] + ["<|im_start|>user\nHi there<|im_end|>\n", "a  b   c\n\n\n d", "I'LL don't CAN'T 123456 x1y2",
                          "emoji 🙂 test…", " x", "tail space  ", ""]
    for c in cases:
        assert t.encode(c) == hf.encode(c).ids, c
        assert t.decode(t.encode(c)) == c
    assert t.piece_id("<|im_end|>") == hf.token_to_id("<|im_end|>")
    assert t.is_special(t.piece_id("<|im_end|>"))
    assert t.encode("<|im_end|>", allow_special=False) != [t.piece_id("<|im_end|>")]
    # byte-exact decode of a split multi-byte character
    ids = t.encode("🙂")
    assert t.decode_bytes(ids) == "🙂".encode()
