"""Makes tests/golden/reference_logits.safetensors: last-position float32 logits of the reference project's
own forward pass (ampere_kv.runner.model_forward, its paged non-fused path, on the CPU) for tiny random
models, so that the plain implementation under tests/plain can be compared with the reference's code and
not only with its formulas.

Run once, where the reference checkout is importable:

    REFERENCE_ROOT=/path/to/ampere-kv-engine python tests/golden/make_golden.py

The reference reads weights off a checkpoint-library model object by attribute; a tree of
``types.SimpleNamespace`` with exactly those attributes stands in for it.  Weights come from the plain
implementation's ``random_weights`` (seed 1), token ids from ``torch.Generator().manual_seed(21)``.
The reference has no sliding window, so configuration B is used with its window switched off; its
attention bias is kept (the reference passes biases through as stored).
Each case is fed whole, and again in portions 5/10/rest.
"""

import os
import sys
import types

sys.dont_write_bytecode = True
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
if "REFERENCE_ROOT" in os.environ:      # needed to make the file; the tests import this module for its cases only
    sys.path.insert(0, os.environ["REFERENCE_ROOT"])

import torch  # noqa: E402
from safetensors.torch import save_file  # noqa: E402

import tiny  # noqa: E402
from plain import qwen3_plain as plain  # noqa: E402


def duck_model(w, cfg):
    ns = types.SimpleNamespace
    heads = cfg["num_attention_heads"]
    head_dim = cfg.get("head_dim", cfg["hidden_size"] // heads)
    eps = cfg["rms_norm_eps"]
    lin = lambda name: ns(weight=w[name + ".weight"], bias=w.get(name + ".bias"))
    norm = lambda name: ns(weight=w[name + ".weight"], variance_epsilon=eps)
    layers = []
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        attn = ns(q_proj=lin(f"{p}.self_attn.q_proj"), k_proj=lin(f"{p}.self_attn.k_proj"),
                  v_proj=lin(f"{p}.self_attn.v_proj"), o_proj=lin(f"{p}.self_attn.o_proj"),
                  q_norm=norm(f"{p}.self_attn.q_norm"), k_norm=norm(f"{p}.self_attn.k_norm"),
                  head_dim=head_dim, sliding_window=None)
        mlp = ns(gate_proj=lin(f"{p}.mlp.gate_proj"), up_proj=lin(f"{p}.mlp.up_proj"), down_proj=lin(f"{p}.mlp.down_proj"))
        layers.append(ns(self_attn=attn, mlp=mlp, input_layernorm=norm(f"{p}.input_layernorm"),
                         post_attention_layernorm=norm(f"{p}.post_attention_layernorm")))
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
    return ns(model=ns(embed_tokens=ns(weight=w["model.embed_tokens.weight"]), layers=layers, norm=norm("model.norm")),
              lm_head=ns(weight=head, bias=None),
              config=ns(head_dim=head_dim, num_key_value_heads=cfg.get("num_key_value_heads", heads),
                        rope_theta=cfg["rope_theta"], hidden_act="silu"),
              _ampere_inv_freq=1.0 / (cfg["rope_theta"] ** exponent),
              generation_config=ns(eos_token_id=None))


def reference_last_logits(model, cfg, ids, cuts):
    from ampere_kv import runner
    from ampere_kv.paged_cache import PagedKVCache, PagedKVStorage
    heads = cfg["num_attention_heads"]
    caches = [PagedKVCache(PagedKVStorage(cfg.get("num_key_value_heads", heads),
                                          cfg.get("head_dim", cfg["hidden_size"] // heads), 16, 16,
                                          kv_dtype=torch.float32)) for _ in range(cfg["num_hidden_layers"])]
    start, logits = 0, None
    for n in cuts:
        chunk = torch.tensor([ids[start:start + n]], dtype=torch.long)
        pos = torch.arange(start, start + n).unsqueeze(0)
        logits = runner.model_forward(model, chunk, pos, caches, is_prefill=True, output_logits=True)
        start += n
    return logits[0, 0].float()


def cases():
    g = torch.Generator().manual_seed(21)
    for name in ("A", "B"):
        cfg = tiny.config(name)
        cfg["use_sliding_window"] = False
        ids_all = torch.randint(0, cfg["vocab_size"], (33,), generator=g).tolist()
        for length in (5, 17, 33):
            yield name, cfg, ids_all[:length]


def main():
    out = {}
    for name, cfg, ids in cases():
        w = plain.random_weights(cfg, 1)
        model = duck_model(w, cfg)
        n = len(ids)
        out[f"{name}.len{n}.whole"] = reference_last_logits(model, cfg, ids, [n])
        if n > 15:
            out[f"{name}.len{n}.portions"] = reference_last_logits(model, cfg, ids, [5, 10, n - 15])
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(HERE, "reference_logits.safetensors"))
    print(f"wrote {len(out)} tensors")


if __name__ == "__main__":
    if "REFERENCE_ROOT" not in os.environ:
        sys.exit("set REFERENCE_ROOT to a checkout of the reference project (ampere-kv-engine)")
    main()
