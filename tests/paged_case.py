"""A ragged attention batch over a shuffled page pool, with the plain formula's answer: shared by the kernel tests
and the test of the allocation-free entry point."""

import torch

from plain import qwen3_plain as plain


def dev(t):
    return t.to("cuda")


def status_word():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


class PagedCase:
    """A ragged batch over a shuffled page pool whose unheld pages are NaN."""

    def __init__(self, dtype, nh, nkv, d, page, q_lens, ctx_lens, seed=0, q_tile=16):
        g = torch.Generator().manual_seed(seed)
        self.nh, self.nkv, self.d, self.page = nh, nkv, d, page
        self.q_lens, self.ctx_lens = q_lens, ctx_lens
        pages_per_seq = [(c + page - 1) // page for c in ctx_lens]
        pool = sum(pages_per_seq) + 5
        order = torch.randperm(pool, generator=g).tolist()
        self.k_seq = [torch.randn(c, nkv, d, generator=g).to(dtype) for c in ctx_lens]
        self.v_seq = [torch.randn(c, nkv, d, generator=g).to(dtype) for c in ctx_lens]
        self.q_seq = [torch.randn(n, nh, d, generator=g).to(dtype) for n in q_lens]
        self.k_cache = torch.full((pool, nkv, page, d), float("nan")).to(dtype)
        self.v_cache = self.k_cache.clone()
        width = max(pages_per_seq)
        self.table = torch.full((len(ctx_lens), width), -1, dtype=torch.int32)
        for s in range(len(ctx_lens)):
            for lp in range(pages_per_seq[s]):
                self.table[s, lp] = order.pop()
        self.rewrite_cache()
        cu = [0]
        for n in q_lens:
            cu.append(cu[-1] + n)
        self.cu = torch.tensor(cu, dtype=torch.int32)
        tile_rows = 1 if max(q_lens) == 1 else q_tile
        tiles = [(s, cu[s] + q0, min(tile_rows, n - q0)) for s, n in enumerate(q_lens) for q0 in range(0, n, tile_rows)]
        self.tile_rows = tile_rows
        self.tiles = [torch.tensor([t[i] for t in tiles], dtype=torch.int32) for i in range(3)]

    def rewrite_cache(self):
        """Copies k_seq / v_seq into the pages that the table names (again, after a test changed some keys)."""
        for s, c in enumerate(self.ctx_lens):
            for lp in range((c + self.page - 1) // self.page):
                pp = int(self.table[s, lp])
                lo, hi = lp * self.page, min(c, (lp + 1) * self.page)
                self.k_cache[pp, :, :hi - lo] = self.k_seq[s][lo:hi].transpose(0, 1)
                self.v_cache[pp, :, :hi - lo] = self.v_seq[s][lo:hi].transpose(0, 1)

    def run(self, ops, window=0, splits=1, scale=None, kernel="auto"):
        scale = scale if scale is not None else self.d ** -0.5
        q = torch.cat([x.reshape(x.shape[0], -1) for x in self.q_seq])
        status = status_word()
        out = ops.paged_attention(
            dev(q), dev(self.k_cache), dev(self.v_cache), dev(self.table), dev(self.cu),
            dev(torch.tensor(self.ctx_lens, dtype=torch.int32)), dev(self.tiles[0]), dev(self.tiles[1]),
            dev(self.tiles[2]), num_tiles=len(self.tiles[0]), q_tile=self.tile_rows, num_splits=splits,
            num_heads=self.nh, num_kv_heads=self.nkv, window=window, scale=scale, status=status, kernel=kernel)
        assert int(status.item()) == 0
        return out.float().cpu()

    def reference(self, window=0, scale=None):
        outs = []
        for s, (n, c) in enumerate(zip(self.q_lens, self.ctx_lens)):
            # whole-sequence attention with the queries placed at the last n positions
            q_full = torch.zeros(c, self.nh, self.d)
            q_full[c - n:] = self.q_seq[s].float()
            if scale is not None:
                q_full = q_full * (scale / self.d ** -0.5)
            o = plain.causal_attention(q_full, self.k_seq[s].float(), self.v_seq[s].float(), window or None)
            outs.append(o[c - n:].reshape(n, -1))
        return torch.cat(outs)
