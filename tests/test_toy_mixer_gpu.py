"""A mixer with fixed-size state of its own, defined here in the test, is registered, built into a model
spec, given state slots by the cache manager and stepped, without any change to the package's files.

The toy mixer is a running sum: y_t = W (x_t + sum of x_s for s < t).  Its state after token t must not
depend on how the tokens before t were cut into steps, nor on what else was in the batch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _register():
    from ampere_kv_engine_b200.parts.base import CacheSpec, Mixer, ParamSpec, MIXERS, register_mixer
    if "toy_running_sum" in MIXERS.kinds():
        return

    @register_mixer("toy_running_sum")
    class RunningSum(Mixer):
        def __init__(self, spec, **kw):
            super().__init__(spec, **kw)
            self.weight = None

        def cache_spec(self):
            return CacheSpec(kind="none", state_shape=(self.hidden_size,))

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.hidden_size, self.hidden_size))}

        def load(self, tensors):
            self.weight = tensors["mix.weight"]

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            row = 0
            for n, slot in zip(ctx.q_lens_host, ctx.state_slots_host):
                chunk = x[row:row + n].float()
                running = torch.cumsum(chunk, dim=0) + cache.state[slot]
                out[row:row + n] = (running @ self.weight.float().t()).to(x.dtype)
                cache.state[slot] = running[-1]
                row += n
            return out


def _spec(hidden=48, vocab=97):
    from ampere_kv_engine_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    rope = PartSpec("rope", {"theta": 10000.0, "rotary_dim": 16})
    attn = PartSpec("attention", {"num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qk_norm": True,
                                  "qk_norm_eps": 1e-6, "position_encoding": rope}, "l1.attn")
    norm = lambda name: PartSpec("rmsnorm", {"eps": 1e-6}, name)
    mlp = lambda name: PartSpec("gated_mlp", {"intermediate_size": 64}, name)
    layers = (
        LayerSpec("prenorm", PartSpec("toy_running_sum", {}, "l0.toy"), mlp("l0.mlp"), norm("l0.n1"), norm("l0.n2")),
        LayerSpec("prenorm", attn, mlp("l1.mlp"), norm("l1.n1"), norm("l1.n2")),
    )
    # the toy layer runs twice (shared weights, a state of its own each time); the second attention
    # position reads the first one's cache
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))
    return ModelSpec(hidden_size=hidden, vocab_size=vocab, embedding=PartSpec("token_embedding", {"vocab_size": vocab}, "emb"),
                     layers=layers, schedule=schedule, final_norm=norm("final"),
                     head=PartSpec("linear_head", {"vocab_size": vocab, "tied": True}, "head"), max_position=256)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_state_mixer_is_built_and_stepped(dtype):
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.step import ModelRunner
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.weights.random_init import init_random
    _register()
    model = DecoderModel(_spec(), dtype=dtype, device="cuda")
    assert "l0.toy.mix.weight" in model.param_specs()
    init_random(model, 5)
    runner = ModelRunner(model, page_size=16, num_pages=32, max_seqs=4)
    # four schedule positions: two toy states, one attention cache shared by two positions
    assert [v.state is not None for v in runner.views] == [True, False, True, False]
    assert runner.views[3].k_cache.data_ptr() == runner.views[1].k_cache.data_ptr() and not runner.views[3].writes
    assert len(runner.manager.groups) == 1 and len(runner.manager.groups[0].positions) == 1
    g = torch.Generator().manual_seed(0)
    toks = {k: torch.randint(0, 97, (n,), generator=g).tolist() for k, n in (("a", 40), ("b", 23))}

    def run(cuts: dict[str, list[int]], together: bool):
        seqs = {k: runner.open(k) for k in cuts}
        rows = {k: [] for k in cuts}
        done = {k: 0 for k in cuts}
        order = [[(k, n) for k, ns in cuts.items() if i < len(ns) for n in [ns[i]]] for i in range(max(map(len, cuts.values())))]
        for step in order:
            groups = [step] if together else [[e] for e in step]
            for grp in groups:
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

    whole = run({"a": [40], "b": [23]}, together=False)
    cut = run({"a": [7, 2, 20, 1, 1, 9], "b": [3, 15, 1, 1, 2, 1]}, together=True)
    tol = dict(atol=5e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    for k in whole:
        torch.testing.assert_close(cut[k], whole[k], **tol)
    # state slots are zeroed when a request opens: the same tokens give the same logits again
    again = run({"a": [40], "b": [23]}, together=False)
    for k in whole:
        torch.testing.assert_close(again[k], whole[k], atol=0, rtol=0)
    runner.manager.check_invariants()
