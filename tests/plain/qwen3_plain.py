"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It is written from the formulas of the
reference project (tdkjsmr/ampere-kv-engine); every function cites the file and lines
(paths inside that project) whose arithmetic it restates.  It shares no code with the
package under test: it reads a ``dict`` of tensors keyed by checkpoint name and a
``dict`` of config.json keys, and runs in whatever dtype the tensors have.

The reference has no sliding window (it rejects one at load, ampere_kv/runner.py:39-40).
The ``window`` argument of :func:`causal_attention` extends the reference's mask
``k_pos <= q_pos`` (ampere_kv/kv_cache.py:85-89) by ``k_pos > q_pos - window``; with
``window=None`` it is exactly the reference's mask.
"""

from __future__ import annotations

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last dim (ampere_kv/runner.py:48-57).

    Square-mean and rsqrt in float32, cast back to the input dtype, then times weight.
    """
    xf = x.float()
    mean_square = xf.square().mean(dim=-1, keepdim=True)
    normed = xf * torch.rsqrt(mean_square + eps)
    return normed.to(x.dtype) * weight.to(x.dtype)


def rope_inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """inv_freq[j] = 1 / theta^(2j / D), float32 (ampere_kv/runner.py:41-44)."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim
    return 1.0 / (theta ** exponent)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE over the full head dim (ampere_kv/runner.py:80-98).

    x: [T, heads, D]; positions: [T] absolute.  Angles in float32, duplicated to both
    halves; cos/sin cast to x's dtype; x*cos + rotate_half(x)*sin in x's dtype.
    """
    angles = positions.to(torch.float32)[:, None] * inv_freq.to(positions.device)[None, :]   # [T, D/2]
    angles = torch.cat((angles, angles), dim=-1)                               # [T, D]
    cos = angles.cos().to(x.dtype)[:, None, :]
    sin = angles.sin().to(x.dtype)[:, None, :]
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rotated * sin


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: int | None = None) -> torch.Tensor:
    """Whole-sequence causal GQA attention (ampere_kv/kv_cache.py:76-94).

    q: [T, NH, D]; k, v: [T, NKV, D].  q-head h reads kv-head h // (NH/NKV)
    (repeat_interleave, kv_cache.py:80-83); scores scaled by D**-0.5 (kv_cache.py:93);
    query i sees key j iff j <= i (kv_cache.py:85-89), and j > i - window when a window
    is given.  Softmax in float32, as the reference's own kernel does
    (csrc/paged_decode.cu:166-243).
    """
    tokens, heads, dim = q.shape
    group = heads // k.shape[1]
    kf = k.float().repeat_interleave(group, dim=1)
    vf = v.float().repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q.float(), kf) * dim ** -0.5
    i = torch.arange(tokens, device=q.device)[:, None]
    j = torch.arange(tokens, device=q.device)[None, :]
    visible = j <= i
    if window is not None:
        visible &= j > i - window
    scores = scores.masked_fill(~visible[None], -torch.inf)
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shd->thd", probs, vf)
    return out.to(q.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T + b with W as stored [out, in] (ampere_kv/runner.py:64-66)."""
    return torch.nn.functional.linear(x, weight, bias)


def attention_part(x: torch.Tensor, positions: torch.Tensor, w: dict, prefix: str, *, num_heads: int,
                   num_kv_heads: int, head_dim: int, eps: float, theta: float,
                   window: int | None) -> torch.Tensor:
    """q/k/v projections, per-head QK-norm, RoPE, attention, o_proj
    (ampere_kv/runner.py:60-77, 120-121, 163-165)."""
    bias = lambda name: w.get(f"{prefix}.{name}.bias")
    q = linear(x, w[f"{prefix}.q_proj.weight"], bias("q_proj")).reshape(-1, num_heads, head_dim)
    k = linear(x, w[f"{prefix}.k_proj.weight"], bias("k_proj")).reshape(-1, num_kv_heads, head_dim)
    v = linear(x, w[f"{prefix}.v_proj.weight"], bias("v_proj")).reshape(-1, num_kv_heads, head_dim)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    inv_freq = rope_inverse_frequencies(head_dim, theta)
    q = apply_rope(q, positions, inv_freq)
    k = apply_rope(k, positions, inv_freq)
    out = causal_attention(q, k, v, window)
    return linear(out.reshape(-1, num_heads * head_dim), w[f"{prefix}.o_proj.weight"], bias("o_proj"))


def gated_mlp(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (ampere_kv/runner.py:172-177)."""
    gate = linear(x, w[f"{prefix}.gate_proj.weight"])
    up = linear(x, w[f"{prefix}.up_proj.weight"])
    return linear(torch.nn.functional.silu(gate) * up, w[f"{prefix}.down_proj.weight"])


def layer_windows(config: dict) -> list[int | None]:
    """Window of each layer from config.json: ``layer_types`` if present, else layers
    ``>= max_window_layers`` slide when ``use_sliding_window`` is true.  (The reference
    only ever runs with no window, ampere_kv/runner.py:39-40.)"""
    layers = config["num_hidden_layers"]
    if not config.get("use_sliding_window", False) or config.get("sliding_window") is None:
        return [None] * layers
    types = config.get("layer_types")
    if types is None:
        first = config.get("max_window_layers", layers)
        types = ["sliding_attention" if i >= first else "full_attention" for i in range(layers)]
    return [config["sliding_window"] if t == "sliding_attention" else None for t in types]


def decoder_layer(h: torch.Tensor, positions: torch.Tensor, w: dict, index: int, config: dict,
                  window: int | None) -> torch.Tensor:
    """Pre-norm block: h + attn(norm(h)), then + mlp(norm(.)) (ampere_kv/runner.py:117-121, 156-179)."""
    prefix = f"model.layers.{index}"
    eps = config.get("rms_norm_eps", 1e-6)
    heads = config["num_attention_heads"]
    x = rms_norm(h, w[f"{prefix}.input_layernorm.weight"], eps)
    attn = attention_part(
        x, positions, w, f"{prefix}.self_attn", num_heads=heads,
        num_kv_heads=config.get("num_key_value_heads", heads),
        head_dim=config.get("head_dim", config["hidden_size"] // heads), eps=eps,
        theta=float(config.get("rope_theta", 10000.0)), window=window)
    after_attention = h + attn
    x2 = rms_norm(after_attention, w[f"{prefix}.post_attention_layernorm.weight"], eps)
    return after_attention + gated_mlp(x2, w, f"{prefix}.mlp")


@torch.no_grad()
def forward_logits(w: dict, config: dict, token_ids: list[int]) -> torch.Tensor:
    """Logits at every position of one whole sequence, float32 [T, vocab].

    Embedding gather (ampere_kv/runner.py:282), the layers in order (runner.py:284-288),
    final norm and output head (runner.py:293-297; the reference keeps only the last
    position, this keeps all).  A tied head reuses the embedding (runner.py:297 reads
    ``lm_head.weight``, which is the embedding tensor when tied).
    """
    device = w["model.embed_tokens.weight"].device       # the whole computation runs where the tensors are
    ids = torch.tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(len(token_ids), device=device)
    h = w["model.embed_tokens.weight"][ids]
    windows = layer_windows(config)
    for index in range(config["num_hidden_layers"]):
        h = decoder_layer(h, positions, w, index, config, windows[index])
    normed = rms_norm(h, w["model.norm.weight"], config.get("rms_norm_eps", 1e-6))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(normed, head).float()


def greedy_generate(w: dict, config: dict, prompt: list[int], max_new_tokens: int,
                    eos_ids: tuple[int, ...] = (), ignore_eos: bool = True) -> list[int]:
    """Greedy loop by whole-sequence recomputation (ampere_kv/runner.py:341-370): argmax of the
    last position, stop at EOS (unless ignored) or at the limit."""
    ids = list(prompt)
    out: list[int] = []
    for _ in range(max_new_tokens):
        token = int(forward_logits(w, config, ids)[-1].argmax())
        out.append(token)
        if (not ignore_eos and token in eos_ids):
            break
        ids.append(token)
    return out


# ---------------------------------------------------------------- sampling

_MASK64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    """splitmix64 finaliser (public-domain constant set), on Python ints."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def uniform_from_key(seed: int, stream: int, step: int) -> float:
    """The uniform in [0, 1) that temperature sampling draws for (seed, request stream, step):
    three chained splitmix64 rounds, top 24 bits.  The reference samples greedily only
    (ampere_kv/runner.py:346); temperature sampling and its generator are this project's own."""
    x = _mix64(seed & _MASK64)
    x = _mix64(x ^ (stream & _MASK64))
    x = _mix64(x ^ (step & _MASK64))
    return (x >> 40) / float(1 << 24)


def temperature_cdf(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Cumulative distribution of softmax(logits / T) in float64, [vocab]."""
    p = torch.softmax(logits.double() / temperature, dim=-1)
    return torch.cumsum(p, dim=-1)


def sample_temperature(logits: torch.Tensor, temperature: float, u: float) -> int:
    """Inverse-CDF draw: the first index whose cumulative probability exceeds u."""
    if temperature == 0.0:
        return int(logits.argmax())
    cdf = temperature_cdf(logits, temperature)
    return int(min(int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float64), right=True)),
                   logits.numel() - 1))


# ---------------------------------------------------------------- random weights (tests' own)

def random_weights(config: dict, seed: int, dtype=torch.float32) -> dict:
    """Random tensors by checkpoint name: matrices N(0, 0.02), norm weights 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    heads = config["num_attention_heads"]
    kv = config.get("num_key_value_heads", heads)
    dim = config.get("head_dim", config["hidden_size"] // heads)
    hidden, inter, vocab = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    mat = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(dtype)
    vec = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)
    w = {"model.embed_tokens.weight": mat(vocab, hidden)}
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = vec(hidden)
        w[f"{p}.self_attn.q_proj.weight"] = mat(heads * dim, hidden)
        w[f"{p}.self_attn.k_proj.weight"] = mat(kv * dim, hidden)
        w[f"{p}.self_attn.v_proj.weight"] = mat(kv * dim, hidden)
        w[f"{p}.self_attn.o_proj.weight"] = mat(hidden, heads * dim)
        if config.get("attention_bias", False):
            for name, n in (("q_proj", heads * dim), ("k_proj", kv * dim), ("v_proj", kv * dim), ("o_proj", hidden)):
                w[f"{p}.self_attn.{name}.bias"] = mat(n)
        w[f"{p}.self_attn.q_norm.weight"] = vec(dim)
        w[f"{p}.self_attn.k_norm.weight"] = vec(dim)
        w[f"{p}.post_attention_layernorm.weight"] = vec(hidden)
        w[f"{p}.mlp.gate_proj.weight"] = mat(inter, hidden)
        w[f"{p}.mlp.up_proj.weight"] = mat(inter, hidden)
        w[f"{p}.mlp.down_proj.weight"] = mat(hidden, inter)
    w["model.norm.weight"] = vec(hidden)
    if not config.get("tie_word_embeddings", False):
        w["lm_head.weight"] = mat(vocab, hidden)
    return w
