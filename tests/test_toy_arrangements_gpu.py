"""Three more arrangements the package does not have, defined and registered here without a change to its files:

* an embedding that scales its rows and a head that soft-caps its logits (kinds looked up in the embedding and
  head registries);
* a block with four norms (one before and one after each branch): how many norms a layer has is the block's
  business, it builds its own parts from the roles of the layer spec;
* a mixer whose cache keeps ONE tensor per token (a compressed vector, no separate keys and values): the cache
  spec names what a token stores and the manager gives it pages of that shape.

They are toys, not anyone's architecture.  The model built from them is stepped whole and in portions, alone and
batched, with few pages so that they are used again, and must give the same logits every way."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _register():
    from ampere_kv_engine_b200.kernels import ops
    from ampere_kv_engine_b200.parts import base

    if "toy_scaled_embedding" not in base.EMBEDDINGS.kinds():
        @base.register_embedding("toy_scaled_embedding")
        class ScaledEmbedding(base.Embedding):
            graph_safe = True

            def __init__(self, spec, **kw):
                super().__init__(spec, **kw)
                self.vocab_size, self.scale = int(spec.params["vocab_size"]), float(spec.params["scale"])

            def param_specs(self):
                return {"weight": base.ParamSpec((self.vocab_size, self.hidden_size))}

            def load(self, tensors):
                self.weight = tensors["weight"].contiguous()

            def forward(self, token_ids, ctx):
                return ops.embedding(token_ids, self.weight, status=ctx.status, sampled=ctx.sampled) * self.scale

    if "toy_softcap_head" not in base.HEADS.kinds():
        @base.register_head("toy_softcap_head")
        class SoftcapHead(base.Head):
            graph_safe = True

            def __init__(self, spec, **kw):
                super().__init__(spec, **kw)
                self.vocab_size, self.cap = int(spec.params["vocab_size"]), float(spec.params["cap"])

            def param_specs(self):
                return {"weight": base.ParamSpec((self.vocab_size, self.hidden_size))}

            def load(self, tensors):
                self.weight = tensors["weight"].contiguous()

            def forward(self, x):
                return self.cap * torch.tanh(ops.linear(x, self.weight, out_dtype=torch.float32) / self.cap)

    if "toy_sandwich" not in base.BLOCKS.kinds():
        @base.register_block("toy_sandwich")
        class SandwichBlock(base.Block):
            """h += post1(mixer(pre1(h))); h += post2(feed_forward(pre2(h))): four norms."""

            def __init__(self, layer, **kw):
                super().__init__(layer, **kw)
                self.mixer_norm = self.build_role("mixer_norm")
                self.mixer = self.build_role("mixer")
                self.post_mixer_norm = self.build_role("post_mixer_norm", base.NORMS)
                self.feed_forward_norm = self.build_role("feed_forward_norm")
                self.feed_forward = self.build_role("feed_forward")
                self.post_feed_forward_norm = self.build_role("post_feed_forward_norm", base.NORMS)

            def forward(self, hidden, delta, ctx, cache):
                x = self.mixer_norm.forward(hidden, delta, ctx)
                branch = self.mixer.forward(x, ctx, cache)
                branch = self.post_mixer_norm.forward(branch.float().contiguous(), None, ctx)
                x = self.feed_forward_norm.forward(hidden, branch, ctx)
                branch = self.feed_forward.forward(x, ctx)
                return hidden, self.post_feed_forward_norm.forward(branch.float().contiguous(), None, ctx)

    if "toy_latent_attention" not in base.MIXERS.kinds():
        @base.register_mixer("toy_latent_attention")
        class LatentAttention(base.Mixer):
            """Each token leaves one compressed vector c_t = W_c x_t in the cache.  Heads query the vectors directly:
            out_t = W_o concat_h(softmax_j<=t(q_th . c_j / sqrt(w)) c_j)."""

            def __init__(self, spec, **kw):
                super().__init__(spec, **kw)
                self.width, self.heads = int(spec.params["width"]), int(spec.params["heads"])

            def cache_spec(self):
                return base.CacheSpec(kind="full", tensors=(base.CacheTensor("latent", 1, self.width),))

            def param_specs(self):
                h, w, n = self.hidden_size, self.width, self.heads
                return {"compress.weight": base.ParamSpec((w, h)), "query.weight": base.ParamSpec((n * w, h)),
                        "out.weight": base.ParamSpec((h, n * w))}

            def load(self, tensors):
                self.w = {k: v.float() for k, v in tensors.items()}

            def forward(self, x, ctx, cache):
                group = ctx.groups[cache.group]
                pages = cache.tensors["latent"]                    # [pages, 1, page_size, width]
                assert cache.k_cache is None and cache.v_cache is None
                page_size = cache.page_size
                xf = x.float()
                latent = (xf @ self.w["compress.weight"].t()).to(pages.dtype)
                slots = group.slot_mapping.long()
                pages[slots // page_size, 0, slots % page_size] = latent
                q = (xf @ self.w["query.weight"].t()).view(-1, self.heads, self.width) * 8.0
                out = torch.empty((x.shape[0], self.heads * self.width), dtype=torch.float32, device=x.device)
                row = 0
                for s, (n, ctx_len) in enumerate(zip(ctx.q_lens_host, ctx.ctx_lens_host)):
                    positions = torch.arange(ctx_len, device=x.device)
                    held = group.block_table[s].long()[positions // page_size]
                    keys = pages[held, 0, positions % page_size].float()          # [ctx, width]
                    scores = torch.einsum("thw,jw->thj", q[row:row + n], keys) / math.sqrt(self.width)
                    first = ctx_len - n
                    visible = positions[None, :] <= (first + torch.arange(n, device=x.device))[:, None]
                    scores = scores.masked_fill(~visible[:, None, :], -math.inf)
                    out[row:row + n] = torch.einsum("thj,jw->thw", torch.softmax(scores, -1), keys).reshape(n, -1)
                    row += n
                return (out @ self.w["out.weight"].t()).to(x.dtype)


def _spec(hidden=80, vocab=173):
    from ampere_kv_engine_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    rope = PartSpec("rope", {"theta": 10000.0, "rotary_dim": 16})
    rms = lambda name: PartSpec("rmsnorm", {"eps": 1e-5}, name)
    attn = PartSpec("attention", {"num_heads": 5, "num_kv_heads": 5, "head_dim": 16, "qk_norm": False,
                                  "position_encoding": rope}, "l1.attn")
    layers = (
        LayerSpec("toy_sandwich", mixer=PartSpec("toy_latent_attention", {"width": 24, "heads": 3}, "l0.mix"),
                  feed_forward=PartSpec("gated_mlp", {"intermediate_size": 112}, "l0.mlp"),
                  mixer_norm=rms("l0.pre1"), feed_forward_norm=rms("l0.pre2"),
                  parts={"post_mixer_norm": rms("l0.post1"), "post_feed_forward_norm": rms("l0.post2")}),
        LayerSpec("prenorm", attn, PartSpec("gated_mlp", {"intermediate_size": 96}, "l1.mlp"), rms("l1.n1"), rms("l1.n2")),
    )
    return ModelSpec(hidden_size=hidden, vocab_size=vocab,
                     embedding=PartSpec("toy_scaled_embedding", {"vocab_size": vocab, "scale": math.sqrt(hidden)}, "emb"),
                     layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
                     final_norm=rms("final"),
                     head=PartSpec("toy_softcap_head", {"vocab_size": vocab, "cap": 1.5}, "head"), max_position=512)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding_softcap_head_four_norms_and_a_one_tensor_cache(dtype):
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.step import ModelRunner
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.weights.random_init import init_random
    _register()
    model = DecoderModel(_spec(), dtype=dtype, device="cuda")
    names = model.param_specs()
    assert {"l0.post1.weight", "l0.post2.weight", "l0.mix.compress.weight", "emb.weight", "head.weight"} <= set(names)
    assert len(model.blocks[0].parts()) == 6 and len(model.blocks[1].parts()) == 4
    init_random(model, 3)
    runner = ModelRunner(model, page_size=8, num_pages=24, max_seqs=4)
    # two groups: the latent cache of the toy layer's two appearances, and the attention layer's keys and values
    shapes = sorted((len(g.positions), tuple(sorted(g.storage))) for g in runner.manager.groups)
    assert shapes == [(1, ("k", "v")), (2, ("latent",))]
    latent_group = next(g for g in runner.manager.groups if "latent" in g.storage)
    assert tuple(latent_group.storage["latent"].shape) == (2, 24, 1, 8, 24)
    assert runner.views[0].tensors["latent"].data_ptr() != runner.views[2].tensors["latent"].data_ptr()
    for g in runner.manager.groups:                     # unheld pages must never be read
        for t in g.storage.values():
            t.fill_(float("nan"))
    gen = torch.Generator().manual_seed(8)
    toks = {k: torch.randint(0, 173, (n,), generator=gen).tolist() for k, n in (("a", 61), ("b", 34), ("c", 50))}

    def run(cuts, together):
        seqs = {k: runner.open(k) for k in cuts}
        rows = {k: [] for k in cuts}
        done = {k: 0 for k in cuts}
        for i in range(max(len(v) for v in cuts.values())):
            step = [(k, ns[i]) for k, ns in cuts.items() if i < len(ns)]
            for grp in ([step] if together else [[e] for e in step]):
                entries = [SeqStep(seqs[k], toks[k][done[k]:done[k] + n], list(range(n))) for k, n in grp]
                logits = runner.step(entries).cpu()
                r = 0
                for k, n in grp:
                    rows[k].append(logits[r:r + n])
                    r += n
                    done[k] += n
        runner.raise_on_status()
        for s in seqs.values():
            runner.close(s)
        return {k: torch.cat(v) for k, v in rows.items()}

    whole = {}
    for k in toks:                                       # each alone: 24 pages do not hold all three at once
        whole.update(run({k: [len(toks[k])]}, together=False))
    assert all(bool(torch.isfinite(v).all()) and float(v.abs().max()) <= 1.5 for v in whole.values())
    assert float(max(v.abs().max() for v in whole.values())) > 0.3      # the cap is not the whole story
    cut = run({"a": [9, 2, 30, 1, 1, 18], "b": [2, 15, 13, 1, 1, 2]}, together=True)
    cut.update(run({"c": [7, 40, 1, 2]}, together=True))
    tol = dict(atol=5e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=4e-2, rtol=4e-2)
    for k in whole:
        torch.testing.assert_close(cut[k], whole[k], **tol)
    assert runner.manager.free_pages() == [24, 24]
    runner.manager.check_invariants()
