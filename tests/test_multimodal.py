"""Multimodal prompts: layout arithmetic, embedding injection and three-axis rotary positions through prefill, decode and
the prefix cache."""
import pytest
import torch

from volta_engine_b200.models.dense import DenseConfig, DenseModel
from volta_engine_b200.runtime import multimodal as MM
from volta_engine_b200.runtime.engine import Engine
from volta_engine_b200.runtime.generator import Generator, Request
from volta_engine_b200.runtime.kv_cache import PagedKVCache
from volta_engine_b200.runtime.options import Options
from volta_engine_b200.runtime.prefix_cache import PrefixCache

IMG = 250


def test_layout_positions_and_cache_keys():
    ids, layout = MM.expand_placeholders([5, 6, IMG, 7, IMG, 8], IMG, [(2, 3), (1, 2)], [b"one", b"two"])
    assert ids == [5, 6] + [IMG] * 6 + [7] + [IMG] * 2 + [8] and layout.n_tokens == 12
    p = layout.positions3()
    assert p[:, :2].tolist() == [[0, 1]] * 3
    assert p[0, 2:8].tolist() == [2] * 6 and p[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and p[2, 2:8].tolist() == [2, 3, 4] * 2
    assert p[:, 8].tolist() == [5, 5, 5]                       # text resumes at 2 + max(2, 3)
    assert p[0, 9:11].tolist() == [6, 6] and p[2, 9:11].tolist() == [6, 7] and p[:, 11].tolist() == [8, 8, 8]
    assert layout.delta() == 9 - 12
    a = layout.cache_tokens(ids)
    _, other = MM.expand_placeholders([5, 6, IMG, 7, IMG, 8], IMG, [(2, 3), (1, 2)], [b"one", b"TWO"])
    b = other.cache_tokens(ids)
    assert a[:9] == b[:9] and a[9:11] != b[9:11] and all(t < 0 for t in a[2:8]) and a[8] == 7
    with pytest.raises(ValueError):
        MM.expand_placeholders([IMG], IMG, [(1, 1), (1, 1)])


def _model(dev="cpu"):
    cfg = DenseConfig.tiny(vocab=256)
    cfg.mrope_sections = (4, 6)
    cfg.quant = "bf16"
    return DenseModel(cfg, dev).init_random(seed=0)


class ByteTok:
    eos_ids = [0]

    def decode_bytes(self, ids, skip_special=False):
        return bytes(i & 0xFF for i in ids)

    def encode(self, text, allow_special=True):
        return list(text.encode())


def _mm_request(H, dev="cpu", data=(b"img-a",)):
    g = torch.Generator().manual_seed(7)
    base = torch.randint(1, 240, (30,), generator=g).tolist()
    base[10] = IMG
    ids, layout = MM.expand_placeholders(base, IMG, [(3, 4)], list(data))
    feats = (torch.randn(12, H, generator=torch.Generator().manual_seed(len(data[0]))) * 0.5).to(torch.bfloat16).to(dev)
    return ids, layout, MM.MmPrompt.build(layout, feats)


def test_text_prompt_is_unchanged_by_the_multimodal_path_and_images_change_the_output():
    m = _model()
    plain_cfg = DenseConfig.tiny(vocab=256)
    plain_cfg.quant = "bf16"
    plain = DenseModel(plain_cfg, "cpu").init_random(seed=0)
    text = torch.randint(1, 240, (40,), generator=torch.Generator().manual_seed(1)).tolist()

    def run(model, prompt, mm=None):
        kv = PagedKVCache(model.cfg.n_layers, model.nkv, model.cfg.head_dim, 16, 2, 512, "cpu")
        eng = Engine(model, kv, use_graphs=False, prefill_chunk=16)
        tok = eng.prefill(0, prompt, mm=mm)
        out = [tok]
        for i in range(4):
            out.append(eng.step([out[-1]], [len(prompt) + i], [0])[0])
        return out
    assert run(m, text) == run(plain, text)                     # equal axes: the sectioned rope is the plain rope
    ids, layout, mm = _mm_request(m.cfg.hidden)
    with_img = run(m, ids, mm)
    no_embed = run(m, ids, MM.MmPrompt.build(layout, None))
    as_text = run(m, ids)
    assert with_img != no_embed or with_img != as_text          # embeddings and positions both reach the model
    # chunking does not matter: one chunk vs 16-row chunks
    kv = PagedKVCache(m.cfg.n_layers, m.nkv, m.cfg.head_dim, 16, 2, 512, "cpu")
    eng = Engine(m, kv, use_graphs=False, prefill_chunk=1000)
    assert eng.prefill(0, ids, mm=mm) == with_img[0]


def test_generator_serves_multimodal_requests_and_keys_the_prefix_cache_by_image_content():
    m = _model()
    kv = PagedKVCache(m.cfg.n_layers, m.nkv, m.cfg.head_dim, 40, 2, 512, "cpu")
    eng = Engine(m, kv, use_graphs=False, prefill_chunk=16)
    cache = PrefixCache(64 << 20, None)
    o = Options.resolve({"max_slots": 2, "prefix_interval": 16}, env={})
    g = Generator(eng, ByteTok(), o, prefix_cache=cache, eos_ids=[])
    ids, layout, mm = _mm_request(m.cfg.hidden)
    r1 = g.generate(Request(ids, max_tokens=6, mm=mm, cache_key=layout.cache_tokens(ids)))
    r2 = g.generate(Request(ids, max_tokens=6, mm=mm, cache_key=layout.cache_tokens(ids)))
    assert r1["tokens"] == r2["tokens"] and r2["usage"]["cached_tokens"] >= 16          # same image: snapshot reused
    ids3, layout3, mm3 = _mm_request(m.cfg.hidden, data=(b"img-bb",))
    r3 = g.generate(Request(ids3, max_tokens=6, mm=mm3, cache_key=layout3.cache_tokens(ids3)))
    assert r3["usage"]["cached_tokens"] <= 10                                            # other image: only the text before it
    txt = g.generate(Request([3, 4, 5, 6], max_tokens=3))                                # a text request after it: offset reset
    assert len(txt["tokens"]) == 3 and eng.h_delta[0] == 0 or eng.h_delta[1] == 0


@pytest.mark.gpu
def test_multimodal_prefill_and_decode_gpu_match_cpu():
    dev = torch.device("cuda:0")
    from volta_engine_b200.models.util import to_device
    mg = _model(dev)
    mc = to_device(mg, "cpu")
    ids, layout, mm = _mm_request(mg.cfg.hidden)
    outs = []
    for model, d in ((mg, dev), (mc, "cpu")):
        kv = PagedKVCache(model.cfg.n_layers, model.nkv, model.cfg.head_dim, 16, 2, 512, d)
        eng = Engine(model, kv, prefill_chunk=16)
        tok = eng.prefill(1, ids, mm=mm)
        out = [tok]
        for i in range(6):                                        # graph replays read the slot's rotary offset from memory
            out.append(eng.step([out[-1]], [len(ids) + i], [1])[0])
        outs.append(out)
    assert outs[0] == outs[1]
