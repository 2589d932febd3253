"""Each part of the model alone against the plain functions, and the part interfaces at work: a
toy architecture, defined here, with a mixer that keeps state of its own, a layer run twice and a
run that reads another run's cache, registered, built and stepped without touching the engine."""

import pytest
import torch

import plain_qwen3 as P
from helpers import TOL, assert_row_close, assert_rows_close

DT_NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}

pytestmark = pytest.mark.gpu
DEV = "cuda"


def env(dtype):
    from mini_sglang_b200.parts import BuildEnv
    return BuildEnv(dtype=dtype, device=torch.device(DEV))


class DictSource:
    def __init__(self, tensors, dtype):
        self.t, self.dtype = tensors, dtype

    def fetch(self, name):
        t = self.t[name]
        return t.to(DEV, self.dtype if t.dim() > 1 or self.dtype == torch.float32 else t.dtype)

    def has(self, name):
        return name in self.t

    def close(self):
        pass


def rand_for(part, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, decl in part.tensors().items():
        t = torch.randn(decl.shape, generator=g)
        t = 1 + 0.1 * t if decl.init == "norm" else 0.05 * t
        out[name] = t.to(torch.bfloat16)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from mini_sglang_b200.config import PartSpec
    from mini_sglang_b200.parts import NORMS
    n = NORMS["rmsnorm"](PartSpec("rmsnorm", {"size": 120, "eps": 3e-6}), "blk.norm", env(dtype))
    assert list(n.tensors()) == ["blk.norm.weight"]
    w = rand_for(n, 0, dtype)
    n.load(DictSource(w, dtype))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 120, generator=g).to(dtype)
    res = torch.randn(9, 120, generator=g)
    y = n.forward(x=x.to(DEV), residual=res.to(DEV))
    ref = P.rms_norm(res + x.float(), w["blk.norm.weight"].float(), 3e-6)
    assert_rows_close(y.float().cpu(), ref.to(dtype).float(), DT_NAME[dtype])


def test_rope_part_table():
    from mini_sglang_b200.config import PartSpec
    from mini_sglang_b200.parts import POSITION_ENCODINGS
    r = POSITION_ENCODINGS["rope_neox"](PartSpec("rope_neox", {"head_dim": 48, "rotary_dim": 48, "theta": 50000.0,
                                                               "max_positions": 777}), "", env(torch.float32))
    tab = r.rotary_table().cpu()
    assert tab.shape == (777, 48) and tab.dtype == torch.float32
    cos, sin = P.rope_angles(torch.arange(777), 48, 50000.0, torch.float32)
    torch.testing.assert_close(tab[:, :24], cos, rtol=0, atol=2e-6)
    torch.testing.assert_close(tab[:, 24:], sin, rtol=0, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from mini_sglang_b200.config import PartSpec
    from mini_sglang_b200.parts import FEED_FORWARDS
    f = FEED_FORWARDS["swiglu_mlp"](PartSpec("swiglu_mlp", {"hidden_size": 72, "intermediate_size": 200}), "l.mlp", env(dtype))
    w = rand_for(f, 2, dtype)
    f.load(DictSource(w, dtype))
    x = torch.randn(11, 72, generator=torch.Generator().manual_seed(3)).to(dtype)
    y = f.forward(x.to(DEV), None)
    ref = P.mlp_block(x.float(), {k: v.float() for k, v in w.items()}, "l.mlp.")
    assert_rows_close(y.float().cpu(), ref, DT_NAME[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from mini_sglang_b200.config import PartSpec
    from mini_sglang_b200.parts import EMBEDDINGS, HEADS
    e = EMBEDDINGS["token_embedding"](PartSpec("token_embedding", {"vocab_size": 333, "hidden_size": 40, "name": "emb.w"}), "", env(dtype))
    w = rand_for(e, 4, dtype)
    e.load(DictSource(w, dtype))
    ids = torch.tensor([0, 332, 7, 7], dtype=torch.int32)
    torch.testing.assert_close(e.forward(ids.to(DEV)).cpu(), w["emb.w"].float()[ids.long()], rtol=0, atol=0)
    for tied in (True, False):
        h = HEADS["lm_head"](PartSpec("lm_head", {"vocab_size": 333, "hidden_size": 40, "tied": tied, "name": "head.w",
                                                  "tied_to": "emb.w"}), "", env(dtype))
        hw = rand_for(h, 5, dtype)
        h.load(DictSource(hw, dtype), embedding=e)
        x = torch.randn(3, 40, generator=torch.Generator().manual_seed(6)).to(dtype)
        out = h.forward(x.to(DEV))
        assert out.dtype == torch.float32
        W = w["emb.w"] if tied else hw["head.w"]
        assert_rows_close(out.cpu(), x.float() @ W.float().T, DT_NAME[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 5])
def test_attention_mixer_part_alone(dtype, window):
    """The mixer with its own projections, norms, rotation and cache write, fed in two portions."""
    from mini_sglang_b200.config import PartSpec
    from mini_sglang_b200.parts import (MIXERS, POSITION_ENCODINGS, GroupContext, KVCacheView, StepContext, Workspace)
    H, nq, nkv, d, Pg = 40, 6, 3, 16, 4
    rope = POSITION_ENCODINGS["rope_neox"](PartSpec("rope_neox", {"head_dim": d, "theta": 1e4, "max_positions": 64}), "", env(dtype))
    m = MIXERS["paged_attention"](PartSpec("paged_attention", {
        "hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d, "scale": d ** -0.5, "qkv_bias": True,
        "qk_norm": True, "qk_norm_eps": 1e-5, "window": window}), "l.self_attn", env(dtype), position=rope)
    w = rand_for(m, 7, dtype)
    m.load(DictSource(w, dtype))
    need = m.cache_need()
    assert (need.n_kv_heads, need.head_dim, need.window) == (nkv, d, window)
    S = 13
    x = torch.randn(S, H, generator=torch.Generator().manual_seed(8)).to(dtype)
    kc = torch.zeros(8, nkv, Pg, d, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    table = torch.tensor([[3, 1, 5, 2]], dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    outs = []
    for s0, s1 in ((0, 6), (6, 13)):
        n = s1 - s0
        pos = list(range(s0, s1))
        loc = [int(table[0, p // Pg]) * Pg + p % Pg for p in pos]
        grp = GroupContext(block_table=table, out_loc=i32(loc), nsplit=None, max_split=1, window=window)
        ctx = StepContext(T=n, B=1, page_size=Pg, input_ids=i32([0] * n), positions=i32(pos), q_start=i32([0, n]),
                          kv_len=i32([s1]), token_req=i32([0] * n), slots=i32([1]), groups=[grp], host_q_lens=[n],
                          host_kv_lens=[s1], host_slots=[1], workspace=Workspace(torch.device(DEV)))
        outs.append(m.forward(x[s0:s1].to(DEV), ctx, KVCacheView(kc, vc, grp, Pg)))
    got = torch.cat(outs).float().cpu()
    # plain: the same block on the whole sequence
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "hidden_size": H, "rms_norm_eps": 1e-5,
           "attention_bias": True, "rope_theta": 1e4}
    wf = {k: v.float() for k, v in w.items()}
    if window is None:
        ref = P.attention_block(x.float(), wf, "l.self_attn.", cfg, torch.arange(S))
    else:
        p = "l.self_attn."
        q = (x.float() @ wf[p + "q_proj.weight"].T + wf[p + "q_proj.bias"]).reshape(S, nq, d)
        k = (x.float() @ wf[p + "k_proj.weight"].T + wf[p + "k_proj.bias"]).reshape(S, nkv, d)
        v = (x.float() @ wf[p + "v_proj.weight"].T + wf[p + "v_proj.bias"]).reshape(S, nkv, d)
        q, k = P.rms_norm(q, wf[p + "q_norm.weight"], 1e-5), P.rms_norm(k, wf[p + "k_norm.weight"], 1e-5)
        cos, sin = P.rope_angles(torch.arange(S), d, 1e4, torch.float32)
        o = P.causal_gqa_attention(P.rope_neox(q, cos, sin), P.rope_neox(k, cos, sin), v, d ** -0.5, window=window)
        ref = o.reshape(S, nq * d) @ wf[p + "o_proj.weight"].T
    assert_rows_close(got, ref, DT_NAME[dtype])


# ---------------------------------------------------------------------------------------
# a toy architecture with a stateful mixer, defined entirely in this test
# ---------------------------------------------------------------------------------------
def _register_toy():
    from mini_sglang_b200.cache import StateNeed
    from mini_sglang_b200.config import ARCHITECTURES, LayerSpec, ModelSpec, PartSpec, Run, register_architecture
    from mini_sglang_b200.parts import MIXERS, Mixer, register_mixer
    from mini_sglang_b200.weights import TensorDecl

    if "running_mean" not in MIXERS:
        @register_mixer("running_mean")
        class RunningMean(Mixer):
            """y_t = W * mean(x_0..x_t): keeps the running sum of its inputs per request as state."""

            def __init__(self, spec, prefix, env, position=None):
                super().__init__(spec, prefix, env)
                self.H = spec["hidden_size"]
                self.w = None

            def tensors(self):
                return {self.name("mix.weight"): TensorDecl((self.H, self.H))}

            def load(self, src):
                self.w = src.fetch(self.name("mix.weight"))

            def cache_need(self):
                return StateNeed((self.H,), "float32")

            def forward(self, x, ctx, cache, writes_cache=True):
                out = torch.empty_like(x)
                t = 0
                for r, n in enumerate(ctx.host_q_lens):
                    slot, n_prev = ctx.host_slots[r], ctx.host_kv_lens[r] - n
                    cs = torch.cumsum(x[t:t + n].float(), 0) + cache.state[slot]
                    cnt = torch.arange(n_prev + 1, n_prev + n + 1, device=x.device, dtype=torch.float32)
                    out[t:t + n] = ((cs / cnt[:, None]) @ self.w.float().T).to(x.dtype)
                    if writes_cache:
                        cache.state[slot] = cs[-1]
                    t += n
                return out

    class ToyConfig:
        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

    def build(cfg):
        r = cfg.raw
        H, V = r["width"], r["vocab"]
        norm = PartSpec("rmsnorm", {"size": H, "eps": r["eps"]})
        ffn = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": r["ffn"]})
        rope = PartSpec("rope_neox", {"head_dim": 16, "theta": 1e4, "max_positions": 256})
        names = {"input": "input_layernorm", "post_mixer": "post_attention_layernorm", "mixer": "self_attn", "feed_forward": "mlp"}
        toy = LayerSpec("toy.layers.0", PartSpec("running_mean", {"hidden_size": H}), ffn,
                        {"input": norm, "post_mixer": norm}, position=None, names=names)
        att = LayerSpec("toy.layers.1", PartSpec("paged_attention", {
            "hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qk_norm": False}), ffn,
            {"input": norm, "post_mixer": norm}, position=rope, names=names)
        # layer 0 runs twice (each run with state of its own), and the last run of the attention
        # layer reads the keys and values its first run wrote
        schedule = [Run(0, cache=0), Run(1, cache=1), Run(0, cache=2), Run(1, cache=1, writes_cache=False)]
        return ModelSpec("ToyStateLM", H, V, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "name": "toy.embed.weight"}),
                         PartSpec("rmsnorm", {"size": H, "eps": r["eps"], "name": "toy.norm.weight"}),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True, "name": "toy.head.weight",
                                              "tied_to": "toy.embed.weight"}),
                         [toy, att], schedule, max_context_len=256)

    register_architecture("ToyStateLM", ToyConfig, build)
    return build, ToyConfig


def toy_plain(w, tokens, eps):
    """Whole sequence, float32, no cache: the toy model's formulas restated."""
    f = {k: v.float() for k, v in w.items()}
    S = len(tokens)
    res = f["toy.embed.weight"][torch.tensor(tokens)]
    cnt = torch.arange(1, S + 1, dtype=torch.float32)[:, None]

    def toy_layer(res):
        y = P.rms_norm(res, f["toy.layers.0.input_layernorm.weight"], eps)
        res = res + (torch.cumsum(y, 0) / cnt) @ f["toy.layers.0.self_attn.mix.weight"].T
        y = P.rms_norm(res, f["toy.layers.0.post_attention_layernorm.weight"], eps)
        return res + P.mlp_block(y, f, "toy.layers.0.mlp.")

    def qkv(y):
        p = "toy.layers.1.self_attn."
        q = (y @ f[p + "q_proj.weight"].T).reshape(S, 4, 16)
        k = (y @ f[p + "k_proj.weight"].T).reshape(S, 2, 16)
        v = (y @ f[p + "v_proj.weight"].T).reshape(S, 2, 16)
        cos, sin = P.rope_angles(torch.arange(S), 16, 1e4, torch.float32)
        return P.rope_neox(q, cos, sin), P.rope_neox(k, cos, sin), v

    def att_layer(res, kv=None):
        y = P.rms_norm(res, f["toy.layers.1.input_layernorm.weight"], eps)
        q, k, v = qkv(y)
        if kv is not None:
            k, v = kv
        o = P.causal_gqa_attention(q, k, v, 16 ** -0.5).reshape(S, 64) @ f["toy.layers.1.self_attn.o_proj.weight"].T
        res = res + o
        y = P.rms_norm(res, f["toy.layers.1.post_attention_layernorm.weight"], eps)
        return res + P.mlp_block(y, f, "toy.layers.1.mlp."), (k, v)

    res = toy_layer(res)
    res, kv = att_layer(res)
    res = toy_layer(res)
    res, _ = att_layer(res, kv)
    return P.rms_norm(res, f["toy.norm.weight"], eps) @ f["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_state_is_registered_built_and_stepped(dtype):
    from mini_sglang_b200.cache import PagedKVNeed, StateNeed
    from mini_sglang_b200.config import ARCHITECTURES
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.weights import RandomSource

    build, Cfg = _register_toy()
    try:
        spec = build(Cfg({"width": 40, "vocab": 97, "ffn": 56, "eps": 1e-5}))
        spec.validate()
        holder = {}

        def factory(expected, dt, dev):
            src = RandomSource(expected, 11, dt, dev, std=0.08)
            holder["w"] = {n: src.draw(n).cpu() for n in expected if src.has(n)}
            return src

        runner = ModelRunner(spec, factory, dtype=dtype, page_size=4, num_pages=32, max_reqs=3, max_step_tokens=64)
        needs = runner.mgr.needs
        assert isinstance(needs[0], StateNeed) and isinstance(needs[1], PagedKVNeed) and isinstance(needs[2], StateNeed)
        assert not runner.use_cuda_graph                      # the toy mixer loops on the host
        g = torch.Generator().manual_seed(5)
        a = torch.randint(0, 97, (29,), generator=g).tolist()
        b = torch.randint(0, 97, (17,), generator=g).tolist()
        sa, sb = runner.open(), runner.open()
        got = {}
        # portions of a beside portions and single tokens of b
        plan = [((0, 7), (0, 5)), ((7, 9), (5, 6)), ((9, 20), (6, 7)), ((20, 29), (7, 17))]
        for (a0, a1), (b0, b1) in plan:
            out = runner.step([StepEntry(sa, a[a0:a1], list(range(a1 - a0))), StepEntry(sb, b[b0:b1], list(range(b1 - b0)))])
            out = out.float().cpu()
            for i in range(a1 - a0):
                got[("a", a0 + i)] = out[i]
            for i in range(b1 - b0):
                got[("b", b0 + i)] = out[a1 - a0 + i]
        runner.close(sa)
        # the slot is taken again: its state rows must start from zero
        runner.open()                                              # slots are handed out first-in first-out
        sc = runner.open()
        assert sc == sa
        out = runner.step([StepEntry(sc, b, list(range(len(b))))]).float().cpu()
        ref_a, ref_b = toy_plain(holder["w"], a, 1e-5), toy_plain(holder["w"], b, 1e-5)
        for (rid, pos), row in got.items():
            assert_row_close(row, (ref_a if rid == "a" else ref_b)[pos], dtype)
        assert_rows_close(out, ref_b, dtype)
    finally:
        ARCHITECTURES.pop("ToyStateLM", None)


# ---------------------------------------------------------------------------------------
# a second toy architecture, again defined entirely in this test: a feed-forward that routes
# every token to one of three experts, and a rotary position encoding of another kind
# (frequencies that grow linearly, over the first 8 of 16 head elements only)
# ---------------------------------------------------------------------------------------
def _register_routed_toy():
    from mini_sglang_b200.config import LayerSpec, ModelSpec, PartSpec, Run, register_architecture
    from mini_sglang_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding
    from mini_sglang_b200.parts import register_feed_forward, register_position_encoding
    from mini_sglang_b200.weights import TensorDecl

    if "toy_top1_experts" not in FEED_FORWARDS:
        @register_feed_forward("toy_top1_experts")
        class Top1Experts(FeedForward):
            """router logits in float32 -> the best expert of E for every token -> gelu MLP of that expert,
            weighted by the router's softmax probability of the chosen expert."""

            graph_safe = False               # gathers the rows of each expert: shapes depend on the tokens

            def __init__(self, spec, prefix, env):
                super().__init__(spec, prefix, env)
                self.H, self.I, self.E = spec["hidden_size"], spec["intermediate_size"], spec["experts"]

            def tensors(self):
                t = {self.name("router.weight"): TensorDecl((self.E, self.H))}
                for e in range(self.E):
                    t[self.name(f"experts.{e}.up.weight")] = TensorDecl((self.I, self.H))
                    t[self.name(f"experts.{e}.down.weight")] = TensorDecl((self.H, self.I))
                return t

            def load(self, src):
                self.router = src.fetch(self.name("router.weight")).float()
                self.up = [src.fetch(self.name(f"experts.{e}.up.weight")) for e in range(self.E)]
                self.down = [src.fetch(self.name(f"experts.{e}.down.weight")) for e in range(self.E)]

            def forward(self, x, ctx):
                logits = x.float() @ self.router.T                        # routing in 32-bit
                prob, best = torch.softmax(logits, -1).max(-1)
                out = torch.zeros_like(x)
                for e in range(self.E):
                    rows = (best == e).nonzero().flatten()
                    if rows.numel():
                        h = torch.nn.functional.gelu(x[rows] @ self.up[e].T)
                        out[rows] = ((h @ self.down[e].T).float() * prob[rows, None]).to(x.dtype)
                return out

    if "toy_linear_rotary" not in POSITION_ENCODINGS:
        @register_position_encoding("toy_linear_rotary")
        class LinearRotary(PositionEncoding):
            """angle(p, i) = p * step * (i + 1) over the first `rot` elements of a head, rotated in halves or, with
            the parameter `interleaved`, in neighbouring pairs."""

            def __init__(self, spec, prefix, env):
                super().__init__(spec, prefix, env)
                self.interleaved = bool(spec.get("interleaved", False))
                p = torch.arange(spec["max_positions"], dtype=torch.float32)[:, None]
                ang = p * spec["step"] * torch.arange(1, spec["rot"] // 2 + 1, dtype=torch.float32)[None, :]
                self.table = torch.cat((ang.cos(), ang.sin()), -1).contiguous().to(env.device)

            def rotary_table(self):
                return self.table

    class Cfg:
        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

    def build(cfg):
        r = cfg.raw
        H, V = r["width"], r["vocab"]
        norm = PartSpec("rmsnorm", {"size": H, "eps": r["eps"]})
        routed = PartSpec("toy_top1_experts", {"hidden_size": H, "intermediate_size": r["ffn"], "experts": 3})
        dense = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": r["ffn"]})
        pos = PartSpec("toy_linear_rotary", {"rot": 8, "step": r["step"], "max_positions": 128})
        pos_pairs = PartSpec("toy_linear_rotary", {"rot": 8, "step": r["step"], "max_positions": 128, "interleaved": True})
        att = lambda window: PartSpec("paged_attention", {"hidden_size": H, "num_heads": 6, "num_kv_heads": 3, "head_dim": 16,  # noqa: E731
                                                          "qk_norm": True, "qk_norm_eps": r["eps"], "window": window})
        # the checkpoint's names of a layer's parts are data: layer 0 has names of its own, layer 1 none (the roles' names)
        layers = [LayerSpec("toy.layers.0", att(None), routed, {"input": norm, "post_mixer": norm}, position=pos,
                            names={"input": "ln1", "post_mixer": "ln2", "mixer": "attn", "feed_forward": "moe"}),
                  LayerSpec("toy.layers.1", att(6), dense, {"input": norm, "post_mixer": norm}, position=pos_pairs)]
        return ModelSpec("ToyRoutedLM", H, V, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "name": "toy.embed.weight"}),
                         PartSpec("rmsnorm", {"size": H, "eps": r["eps"], "name": "toy.norm.weight"}),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": False, "name": "toy.head.weight"}),
                         layers, [Run(0, cache=0), Run(1, cache=1)], max_context_len=128)

    register_architecture("ToyRoutedLM", Cfg, build)
    return build, Cfg


def routed_toy_plain(w, tokens, eps, step):
    f = {k: v.float() for k, v in w.items()}
    S = len(tokens)
    res = f["toy.embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(S, dtype=torch.float32)[:, None]
    ang = pos * step * torch.arange(1, 5, dtype=torch.float32)[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rotate(x, pairs):                            # first 8 elements of every head
        if pairs:                                    # neighbours 2 p, 2 p + 1 (layer 1)
            a, b, rest = x[..., 0:8:2], x[..., 1:8:2], x[..., 8:]
            return torch.cat((torch.stack((a * cos - b * sin, b * cos + a * sin), -1).flatten(-2), rest), -1)
        a, b, rest = x[..., :4], x[..., 4:8], x[..., 8:]          # halves of 4 against each other (layer 0)
        return torch.cat((a * cos - b * sin, b * cos + a * sin, rest), -1)

    def attention(y, p, window):
        pairs = window is not None
        q = P.rms_norm((y @ f[p + "q_proj.weight"].T).reshape(S, 6, 16), f[p + "q_norm.weight"], eps)
        k = P.rms_norm((y @ f[p + "k_proj.weight"].T).reshape(S, 3, 16), f[p + "k_norm.weight"], eps)
        v = (y @ f[p + "v_proj.weight"].T).reshape(S, 3, 16)
        q, k = rotate(q, pairs), rotate(k, pairs)
        k, v = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * 16 ** -0.5
        i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
        ok = (j <= i) if window is None else ((j <= i) & (j > i - window))
        s = s.masked_fill(~ok, float("-inf"))
        return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(S, 96) @ f[p + "o_proj.weight"].T

    def experts(y, p):
        prob, best = torch.softmax(y @ f[p + "router.weight"].T, -1).max(-1)
        out = torch.zeros_like(y)
        for e in range(3):
            rows = (best == e).nonzero().flatten()
            out[rows] = (torch.nn.functional.gelu(y[rows] @ f[p + f"experts.{e}.up.weight"].T) @ f[p + f"experts.{e}.down.weight"].T) * prob[rows, None]
        return out, best

    y = P.rms_norm(res, f["toy.layers.0.ln1.weight"], eps)
    res = res + attention(y, "toy.layers.0.attn.", None)
    y = P.rms_norm(res, f["toy.layers.0.ln2.weight"], eps)
    moe, best = experts(y, "toy.layers.0.moe.")
    res = res + moe
    y = P.rms_norm(res, f["toy.layers.1.input.weight"], eps)
    res = res + attention(y, "toy.layers.1.mixer.", 6)
    y = P.rms_norm(res, f["toy.layers.1.post_mixer.weight"], eps)
    res = res + P.mlp_block(y, f, "toy.layers.1.feed_forward.")
    return P.rms_norm(res, f["toy.norm.weight"], eps) @ f["toy.head.weight"].T, best


def test_toy_architecture_with_routed_experts_and_another_rotary_encoding():
    """Registered, built and stepped without a change to the framework's files: a feed-forward with routing, a
    rotary encoding of another kind with partial rotation (in halves in one layer, in neighbouring pairs in the other),
    layers that differ in feed-forward, window and position encoding."""
    from mini_sglang_b200.config import ARCHITECTURES
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.weights import RandomSource

    build, Cfg = _register_routed_toy()
    try:
        spec = build(Cfg({"width": 48, "vocab": 83, "ffn": 40, "eps": 1e-5, "step": 0.07}))
        spec.validate()
        holder = {}

        def factory(expected, dt, dev):
            src = RandomSource(expected, 23, dt, dev, std=0.15)
            holder["w"] = {n: src.draw(n).cpu() for n in expected if src.has(n)}
            return src

        runner = ModelRunner(spec, factory, dtype="float32", page_size=4, num_pages=24, max_reqs=2, max_step_tokens=64)
        assert len(runner.mgr.groups) == 2                    # all keys / a window of 6: pages of their own
        assert not runner.use_cuda_graph
        g = torch.Generator().manual_seed(8)
        toks = torch.randint(0, 83, (37,), generator=g).tolist()
        ref, best = routed_toy_plain(holder["w"], toks, 1e-5, 0.07)
        assert len(set(best.tolist())) == 3                   # every expert gets tokens
        s = runner.open()
        got = []
        for lo, hi in [(0, 9), (9, 11), (11, 30), (30, 31), (31, 37)]:
            got.append(runner.step([StepEntry(s, toks[lo:hi], list(range(hi - lo)))]).float().cpu())
        torch.testing.assert_close(torch.cat(got), ref, **TOL["float32"])
    finally:
        ARCHITECTURES.pop("ToyRoutedLM", None)


def test_scheduler_runs_a_toy_model_with_two_cache_groups_under_a_small_pool():
    """The scheduler above the real step function of a model it knows nothing about: routed experts, a layer that keeps all
    keys and a layer that keeps a window of 6 (two cache groups with pools of their own), prompts fed 8 tokens a step, and so
    few pages that requests have to wait for one another.  Greedy tokens equal those of the toy's plain restatement; nothing is
    left in either pool."""
    from mini_sglang_b200.config import ARCHITECTURES
    from mini_sglang_b200.engine.scheduler import Req, Scheduler
    from mini_sglang_b200.engine.step import ModelRunner
    from mini_sglang_b200.sampling import Sampler, SamplingParams
    from mini_sglang_b200.weights import RandomSource

    build, Cfg = _register_routed_toy()
    try:
        spec = build(Cfg({"width": 48, "vocab": 83, "ffn": 40, "eps": 1e-5, "step": 0.07}))
        holder = {}

        def factory(expected, dt, dev):
            src = RandomSource(expected, 23, dt, dev, std=0.15)
            holder["w"] = {n: src.draw(n).cpu() for n in expected if src.has(n)}
            return src

        runner = ModelRunner(spec, factory, dtype="float32", page_size=4, num_pages=22, max_reqs=4, max_step_tokens=32)
        assert len(runner.mgr.groups) == 2
        sch = Scheduler(runner, Sampler(0, runner.device), max_num_reqs=4, max_step_tokens=32, chunk_size=8, policy="lpm",
                        retract_decode_steps=2)
        assert sch.tree is None and sch.policy == "fcfs"      # no prefix sharing for a model with a windowed group
        g = torch.Generator().manual_seed(9)
        prompts = [torch.randint(0, 83, (n,), generator=g).tolist() for n in (19, 7, 26, 11, 15)]
        n_new = 9
        reqs = [Req(f"r{i}", p, SamplingParams(max_new_tokens=n_new, ignore_eos=True)) for i, p in enumerate(prompts)]
        for r in reqs:
            sch.add_request(r)
        most_running = 0
        for _ in range(2000):
            if sch.idle:
                break
            sch.step()
            most_running = max(most_running, len(sch.running))
        assert sch.idle and most_running >= 2
        sch.check_idle_invariants()
        assert all(gr.pool.in_use == 0 for gr in runner.mgr.groups)
        for r, p in zip(reqs, prompts):
            assert r.finish_reason.type == "length" and len(r.output) == n_new
            toks = list(p)
            for t in r.output:                                 # greedy under the plain restatement, given the same history
                ref, _ = routed_toy_plain(holder["w"], toks, 1e-5, 0.07)
                top2 = ref[-1].topk(2).values
                if top2[0] - top2[1] > 1e-4:
                    assert int(ref[-1].argmax()) == t, (r.rid, len(toks) - len(p))
                toks.append(t)
    finally:
        ARCHITECTURES.pop("ToyRoutedLM", None)


# ---------------------------------------------------------------------------------------
# a third toy architecture, defined here as well: a norm of another kind (mean-centred, with a bias)
# and another arrangement of a block (one norm, mixer and feed-forward side by side on its output)
# ---------------------------------------------------------------------------------------
def _register_parallel_toy():
    from mini_sglang_b200.config import LayerSpec, ModelSpec, PartSpec, Run, register_architecture
    from mini_sglang_b200.parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, Norm, Part, build_part
    from mini_sglang_b200.parts import register_block, register_embedding, register_head, register_norm
    from mini_sglang_b200.weights import TensorDecl

    if "toy_token_and_place" not in EMBEDDINGS:
        @register_embedding("toy_token_and_place")
        class TokenAndPlace(Part):
            """h = E[id] + A[position]: a position encoding that is added to the hidden state (a learned vector for every
            place) belongs to the embedding part, which gets the step's context for it."""

            def __init__(self, spec, prefix, env):
                super().__init__(spec, prefix, env)
                self.V, self.H, self.places = spec["vocab_size"], spec["hidden_size"], spec["places"]
                self.tensor_name, self.place_name = spec["name"], spec["place_name"]

            def tensors(self):
                return {self.tensor_name: TensorDecl((self.V, self.H)), self.place_name: TensorDecl((self.places, self.H))}

            def load(self, src):
                self.weight, self.place = src.fetch(self.tensor_name).contiguous(), src.fetch(self.place_name).contiguous()

            def forward(self, ids, ctx=None):
                return self.weight[ids.long()].float() + self.place[ctx.positions.long()].float()

    if "toy_capped_head" not in HEADS:
        @register_head("toy_capped_head")
        class CappedHead(Part):
            """logits = cap * tanh((h W^T + bias) / cap), float32: an output head with a bias and a soft cap."""

            def __init__(self, spec, prefix, env):
                super().__init__(spec, prefix, env)
                self.V, self.H, self.cap = spec["vocab_size"], spec["hidden_size"], spec["cap"]

            def tensors(self):
                return {"toy.head.weight": TensorDecl((self.V, self.H)), "toy.head.bias": TensorDecl((self.V,), kind="vector")}

            def load(self, src, embedding=None):
                self.weight, self.bias = src.fetch("toy.head.weight").contiguous(), src.fetch("toy.head.bias").float()

            def forward(self, h):
                from mini_sglang_b200 import ops
                return self.cap * torch.tanh((ops.linear(h, self.weight, out_dtype=torch.float32) + self.bias) / self.cap)

    if "toy_centred_norm" not in NORMS:
        @register_norm("toy_centred_norm")
        class CentredNorm(Norm):
            """v = residual + x; y = (v - mean(v)) * rsqrt(var(v) + eps) * weight + bias, in float32.  The sum goes to
            `residual_out`; `rows` picks the rows that are normed."""

            def __init__(self, spec, prefix, env):
                super().__init__(spec, prefix, env)
                self.size, self.eps = spec["size"], spec["eps"]
                self.w_name, self.b_name = spec.get("name", self.name("weight")), spec.get("bias_name", self.name("bias"))

            def tensors(self):
                return {self.w_name: TensorDecl((self.size,), kind="vector", init="norm"),
                        self.b_name: TensorDecl((self.size,), kind="vector")}

            def load(self, src):
                self.weight, self.bias = src.fetch(self.w_name).float(), src.fetch(self.b_name).float()

            def forward(self, x=None, residual=None, residual_out=None, rows=None):
                v = residual if x is None else (x.float() if residual is None else residual + x.float())
                if residual_out is not None and x is not None:
                    residual_out.copy_(v)
                if rows is not None:
                    v = v[rows.long()]
                c = v - v.mean(-1, keepdim=True)
                y = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight + self.bias
                return y.to(self.env.dtype)

    if "toy_side_by_side" not in BLOCKS:
        @register_block("toy_side_by_side")
        class SideBySideBlock(Block):
            """res += delta_in; y = norm(res); delta_out = mixer(y) + feed_forward(y): one norm a layer, both branches
            read its output.  The engine asks a block for `mixer` (cache need, graph safety) and `ffn` (graph safety)."""

            def __init__(self, layer_spec, env):
                super().__init__(None, layer_spec.prefix, env)
                at = layer_spec.part_prefix
                self.position = None
                if layer_spec.position is not None:
                    self.position = env.shared(layer_spec.position, lambda: build_part(
                        POSITION_ENCODINGS, "position encoding", layer_spec.position, layer_spec.prefix, env))
                self.norm = build_part(NORMS, "norm", layer_spec.norms["input"], at("input"), env)
                self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, at("mixer"), env, position=self.position)
                self.ffn = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, at("feed_forward"), env)

            def parts(self):
                return [p for p in (self.position, self.norm, self.mixer, self.ffn) if p is not None]

            def tensors(self):
                out = {}
                for part in self.parts():
                    out.update(part.tensors())
                return out

            def load(self, src):
                for part in self.parts():
                    part.load(src)

            def forward(self, delta, residual, ctx, cache, writes_cache=True):
                y = self.norm.forward(x=delta, residual=residual, residual_out=residual if delta is not None else None)
                return self.mixer.forward(y, ctx, cache, writes_cache) + self.ffn.forward(y, ctx), residual

    class Cfg:
        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

    def build(cfg):
        r = cfg.raw
        H, V = r["width"], r["vocab"]
        norm = PartSpec("toy_centred_norm", {"size": H, "eps": r["eps"]})
        pos = PartSpec("rope_neox", {"head_dim": 32, "rotary_dim": 16, "theta": 500.0, "max_positions": 256})
        att = PartSpec("paged_attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 32, "qk_norm": False})
        ffn = PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": r["ffn"]})
        # layer 0 rotates q and k, layer 1 has no position encoding of its own (the places are in the stream already)
        layers = [LayerSpec(f"toy.h.{i}", att, ffn, {"input": norm}, position=pos if i == 0 else None, block="toy_side_by_side",
                            names={"input": "ln", "mixer": "attn", "feed_forward": "mlp"}) for i in range(2)]
        return ModelSpec("ToySideBySideLM", H, V,
                         PartSpec("toy_token_and_place", {"vocab_size": V, "hidden_size": H, "places": 256, "name": "toy.wte.weight",
                                                          "place_name": "toy.wpe.weight"}),
                         PartSpec("toy_centred_norm", {"size": H, "eps": r["eps"], "name": "toy.ln_f.weight", "bias_name": "toy.ln_f.bias"}),
                         PartSpec("toy_capped_head", {"vocab_size": V, "hidden_size": H, "cap": 2.0}),
                         layers, [Run(0, cache=0), Run(1, cache=1)], max_context_len=256)

    register_architecture("ToySideBySideLM", Cfg, build)
    return build, Cfg


def side_by_side_plain(w, tokens, eps):
    f = {k: v.float() for k, v in w.items()}
    S = len(tokens)
    res = f["toy.wte.weight"][torch.tensor(tokens)] + f["toy.wpe.weight"][:S]
    inv = 1.0 / (500.0 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def norm(v, p):
        c = v - v.mean(-1, keepdim=True)
        return c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * f[p + "weight"] + f[p + "bias"]

    def rotate(x):                                   # the first 16 of a head's 32 elements, in halves of 8
        a, b, rest = x[..., :8], x[..., 8:16], x[..., 16:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin, rest), -1)

    for i in range(2):
        p = f"toy.h.{i}."
        y = norm(res, p + "ln.")
        q = (y @ f[p + "attn.q_proj.weight"].T).reshape(S, 4, 32)
        k = (y @ f[p + "attn.k_proj.weight"].T).reshape(S, 2, 32)
        if i == 0:
            q, k = rotate(q), rotate(k)
        k = k.repeat_interleave(2, 1)
        v = (y @ f[p + "attn.v_proj.weight"].T).reshape(S, 2, 32).repeat_interleave(2, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * 32 ** -0.5
        s = s.masked_fill(~(torch.arange(S)[None, :] <= torch.arange(S)[:, None]), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(S, 128) @ f[p + "attn.o_proj.weight"].T
        res = res + a + P.mlp_block(y, f, p + "mlp.")
    return 2.0 * torch.tanh((norm(res, "toy.ln_f.") @ f["toy.head.weight"].T + f["toy.head.bias"]) / 2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_norm_and_a_block_arrangement_of_its_own(dtype):
    """Registered, built and stepped without a change to the framework's files: an embedding that adds a learned vector
    for every place, a mean-centred norm with a bias (also as the model's final norm, on the wanted rows only), a block
    with one norm whose output the mixer and the feed-forward read side by side, and an output head with a bias and a soft
    cap; one layer rotates q and k, the other has no position encoding.  A prompt whole, another in portions, then both decoded token by token through the
    CUDA graph; every row against the toy's plain restatement."""
    from mini_sglang_b200.config import ARCHITECTURES
    from mini_sglang_b200.engine.step import ModelRunner, StepEntry
    from mini_sglang_b200.weights import RandomSource

    build, Cfg = _register_parallel_toy()
    try:
        spec = build(Cfg({"width": 72, "vocab": 131, "ffn": 88, "eps": 1e-5}))
        spec.validate()
        holder = {}

        def factory(expected, dt, dev):
            src = RandomSource(expected, 31, dt, dev, std=0.12)
            holder["w"] = {n: src.draw(n).cpu() for n in expected if src.has(n)}
            return src

        runner = ModelRunner(spec, factory, dtype=dtype, page_size=8, num_pages=24, max_reqs=2, max_step_tokens=64)
        assert runner.use_cuda_graph and len(runner.mgr.groups) == 1
        g = torch.Generator().manual_seed(12)
        a = torch.randint(0, 131, (45,), generator=g).tolist()
        b = torch.randint(0, 131, (38,), generator=g).tolist()
        sa, sb = runner.open(), runner.open()
        got = {}

        def step(parts):                             # parts: [(name, slot, tokens, first position)]
            out = runner.step([StepEntry(s, t, list(range(len(t)))) for _, s, t, _ in parts]).float().cpu()
            i = 0
            for name, _, t, p0 in parts:
                for k in range(len(t)):
                    got[(name, p0 + k)] = out[i]
                    i += 1

        step([("a", sa, a[:40], 0)])
        step([("b", sb, b[:9], 0)])
        step([("b", sb, b[9:11], 9)])
        step([("b", sb, b[11:33], 11)])
        for k in range(5):
            step([("a", sa, a[40 + k:41 + k], 40 + k), ("b", sb, b[33 + k:34 + k], 33 + k)])
            assert runner.last_step_used_graph
        ref = {"a": side_by_side_plain(holder["w"], a, 1e-5), "b": side_by_side_plain(holder["w"], b, 1e-5)}
        assert len(got) == 45 + 38
        for (name, pos), row in got.items():
            try:
                assert_row_close(row, ref[name][pos], dtype)
            except AssertionError as e:
                raise AssertionError(f"request {name}, position {pos}: {e}") from None
    finally:
        ARCHITECTURES.pop("ToySideBySideLM", None)
