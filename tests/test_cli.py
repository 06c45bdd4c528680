"""Launch configuration (flags > JSON file > ENGINE_* environment > defaults; unknown keys fatal) and a server started
from a model directory the way ``volta_server`` does it."""
import http.client
import json
import os

import pytest

from volta_engine_b200.models.dense import DenseConfig
from volta_engine_b200.models.factory import save_dense_checkpoint
from volta_engine_b200.server.cli import build_server, main, resolve_config
from test_tokenizer import _train


def test_precedence_and_unknown_keys(tmp_path):
    launch = tmp_path / "launch.json"
    launch.write_text(json.dumps({"model_dir": "/m/json", "port": 9001, "tp_size": 2, "default_max_tokens": 77,
                                  "options": {"max_seq": 4096, "prefill_chunk": 512}}))
    env = {"ENGINE_PORT": "7000", "ENGINE_HOST": "0.0.0.0", "ENGINE_MAX_SEQ": "1024", "ENGINE_MAX_SLOTS": "3"}
    cfg, _ = resolve_config([str(launch), "--port", "9100", "--set", "prefill_chunk=256"], env=env)
    assert cfg.port == 9100                      # flag beats file beats env
    assert cfg.host == "0.0.0.0"                 # env beats default
    assert cfg.model_dir == "/m/json" and cfg.default_max_tokens == 77
    assert cfg.tp_size == 2 and cfg.options.tp == 2
    assert cfg.options.max_seq == 4096           # file beats env
    assert cfg.options.max_slots == 3            # env beats default
    assert cfg.options.prefill_chunk == 256      # --set beats file
    cfg2, _ = resolve_config([str(launch), "--tp", "4"], env={})
    assert cfg2.tp_size == 4 and cfg2.options.tp == 4
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"model_type": "qwen3"}))       # the model type is never configured
    with pytest.raises(KeyError):
        resolve_config([str(bad)], env={})
    with pytest.raises(KeyError):
        resolve_config(["--set", "nonsense=1"], env={})
    bad.write_text(json.dumps({"options": {"nonsense": 1}}))
    with pytest.raises(KeyError):
        resolve_config([str(bad)], env={})


def test_print_config_docs_and_missing_model(capsys):
    assert main(["--print-config-docs"]) == 0
    out = capsys.readouterr().out
    assert "| `kv_format` |" in out and "ENGINE_MAX_SEQ" in out
    assert main([]) == 2


def test_server_from_model_directory(tmp_path):
    d = str(tmp_path)
    _train(d)
    with open(os.path.join(d, "tokenizer_config.json"), "w") as f:
        json.dump({"chat_template": "{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}"
                                    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}",
                   "eos_token": "<|im_end|>"}, f)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"temperature": 0.0, "top_k": 1}, f)
    cfg = DenseConfig(n_layers=2, hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=512, vocab=640, qk_norm=True)
    save_dense_checkpoint(d, cfg, seed=1, fmt="nvfp4", std=0.05)
    lc, _ = resolve_config(["--model-dir", d, "--port", "0", "--model-name", "tiny-dir", "--set", "max_seq=512",
                            "--set", "max_slots=2", "--set", "prefill_chunk=64", "--default-max-tokens", "8"], env={})
    srv, gen, eng = build_server(lc, device="cpu")
    srv.start()
    try:
        assert srv.defaults["temperature"] == 0.0 and srv.model_type == "qwen3"
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=120)
        c.request("POST", "/v1/chat/completions", body=json.dumps({"model": "tiny-dir", "messages": [
            {"role": "user", "content": "Hello world"}], "max_tokens": 5}), headers={"Content-Type": "application/json"})
        r = c.getresponse()
        body = json.loads(r.read())
        assert r.status == 200, body
        assert body["usage"]["completion_tokens"] <= 5 and body["model"] == "tiny-dir"
    finally:
        srv.stop()
