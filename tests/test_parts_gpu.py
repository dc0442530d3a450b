"""Each part alone against its plain statement, and the framework's generality: a toy mixer
with state of its own, a toy feed-forward with routing, a toy position encoding and a toy
architecture are defined HERE, registered, built and stepped - no file of the framework
knows them.  They are not models of anyone's."""
from __future__ import annotations

import json
import math
import os

import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make_ctx(dtype, positions, entry_of_token, q_start, kv_len, block_table=None, kv_slot=None, page_size=8, slots=None):
    from reinfer_b200.parts.context import GroupView, StepContext
    T, E = len(positions), len(q_start) - 1
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx = StepContext(dtype=dtype, device=torch.device(DEV), n_tokens=T, n_entries=E,
                      n_decode=sum(1 for e in range(E) if q_start[e + 1] - q_start[e] == 1 and all(
                          q_start[k + 1] - q_start[k] == 1 for k in range(e + 1))),
                      token_ids=i32([0] * T), positions=i32(positions), tok_entry=i32(entry_of_token), cu_q=i32(q_start),
                      kv_len=i32(kv_len), entry_slot=i32(slots or list(range(E))), q_start=list(q_start),
                      start_pos=[kv_len[e] - (q_start[e + 1] - q_start[e]) for e in range(E)], slots=slots or list(range(E)),
                      max_q_len=max(q_start[e + 1] - q_start[e] for e in range(E)), max_kv_len=max(kv_len))
    group = None
    if block_table is not None:
        group = GroupView(page_size=page_size, block_table=i32(block_table), kv_slot=i32(kv_slot),
                          max_pages=len(block_table[0]), window=None)
    return ctx, group


def bind_random(part, dtype, seed=0):
    from reinfer_b200.weights.loader import random_state
    state = random_state(part.param_specs(), seed, dtype, DEV)
    part.bind(state)
    return state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from reinfer_b200.parts.norm import RMSNorm
    n = RMSNorm(width=200, eps=1e-4)
    w = bind_random(n, dtype)["weight"]
    ctx, _ = make_ctx(dtype, [0, 1, 2], [0, 0, 0], [0, 3], [3])
    x = torch.randn(3, 200, device=DEV)
    out = n.forward(ctx, x)
    ref = plain.rms_norm(x.double(), w.double(), 1e-4)
    assert out.dtype == dtype
    assert (out.double() - ref).abs().max().item() <= (1e-2 if dtype == torch.bfloat16 else 1e-5) * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_adds_into_residual(dtype):
    from reinfer_b200.parts.ffn import SwiGLU
    f = SwiGLU(hidden=96, intermediate=160)
    st = bind_random(f, dtype)
    ctx, _ = make_ctx(dtype, list(range(5)), [0] * 5, [0, 5], [5])
    xn = torch.randn(5, 96, device=DEV).to(dtype)
    res = torch.randn(5, 96, device=DEV)
    before = res.clone()
    f.forward(ctx, xn, res)
    ref = plain.swiglu_ffn(xn.double(), st["gate_proj.weight"].double(), st["up_proj.weight"].double(),
                           st["down_proj.weight"].double())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert ((res - before).double() - ref).abs().max().item() <= tol * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from reinfer_b200.parts.embedding import Embedding, LMHead
    emb, head = Embedding(vocab=311, hidden=96), LMHead(vocab=311, hidden=96)
    table = bind_random(emb, dtype)["weight"]
    w = bind_random(head, dtype, seed=1)["weight"]
    ctx, _ = make_ctx(dtype, [0, 1, 2, 3], [0] * 4, [0, 4], [4])
    ctx.token_ids = torch.tensor([3, 310, 0, 3], dtype=torch.int32, device=DEV)
    x = emb.forward(ctx)
    assert x.dtype == torch.float32 and torch.equal(x, table[ctx.token_ids.long()].float())
    rows = x[:2].to(dtype).contiguous()
    logits = head.forward(ctx, rows)
    assert logits.dtype == torch.float32
    ref = rows.double() @ w.double().t()
    assert (logits.double() - ref).abs().max().item() <= 1e-3 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("qk_norm", [True, False])
def test_attention_part_whole_and_continued(dtype, qk_norm):
    """The mixer alone: one request whole, then the same request in two steps (the second
    continues from cached pages) beside a second request; compared with the plain block."""
    from reinfer_b200.parts.attention import Attention
    from reinfer_b200.parts.context import LayerCache
    h, QH, KH, d, page = 96, 6, 2, 32, 8
    att = Attention(hidden=h, q_heads=QH, kv_heads=KH, head_dim=d, qk_norm=qk_norm, qk_norm_eps=1e-5,
                    position={"kind": "rope", "head_dim": d, "theta": 1e4})
    st = bind_random(att, dtype, seed=3)
    att.prepare(DEV, dtype)
    S = 21
    xn = (torch.randn(S, h, device=DEV) * 0.5).to(dtype)
    cfg = dict(num_attention_heads=QH, num_key_value_heads=KH, head_dim=d, rms_norm_eps=1e-5, rope_theta=1e4, hidden_size=h)
    w = {"p." + k: v.double().cpu() for k, v in st.items()}
    if not qk_norm:
        w["p.q_norm.weight"] = torch.ones(d, dtype=torch.float64)
        w["p.k_norm.weight"] = torch.ones(d, dtype=torch.float64)
        # without the head norm the plain block must not normalise either: rebuild it from its parts
        def ref_fn(x):
            q = plain.linear(x, w["p.q_proj.weight"]).reshape(-1, QH, d)
            k = plain.linear(x, w["p.k_proj.weight"]).reshape(-1, KH, d)
            v = plain.linear(x, w["p.v_proj.weight"]).reshape(-1, KH, d)
            pos = torch.arange(x.shape[0])
            a = plain.causal_gqa_attention(plain.rope_half_split(q, pos, 1e4), plain.rope_half_split(k, pos, 1e4), v)
            return plain.linear(a.reshape(-1, QH * d), w["p.o_proj.weight"])
    else:
        ref_fn = lambda x: plain.attention_block(x, w, "p.", cfg, torch.arange(x.shape[0]))
    ref = ref_fn(xn.double().cpu())
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
    cache = torch.zeros(8, 2, KH, page, d, dtype=dtype, device=DEV)
    # (1) whole, pages 5,2,7
    ctx, g = make_ctx(dtype, list(range(S)), [0] * S, [0, S], [S], [[5, 2, 7]], [[5, 2, 7][p // page] * page + p % page for p in range(S)], page)
    res = torch.zeros(S, h, device=DEV)
    att.forward(ctx, xn, res, LayerCache(kv=cache, group=g))
    assert (res.double().cpu() - ref).abs().max().item() <= tol * ref.abs().max().item()
    # (2) first 13 tokens, then 8 more beside a one-token request
    cache.zero_()
    ctx, g = make_ctx(dtype, list(range(13)), [0] * 13, [0, 13], [13], [[1, 6, 0]], [[1, 6, 0][p // page] * page + p % page for p in range(13)], page)
    res1 = torch.zeros(13, h, device=DEV)
    att.forward(ctx, xn[:13].contiguous(), res1, LayerCache(kv=cache, group=g))
    other = (torch.randn(1, h, device=DEV) * 0.5).to(dtype)
    ctx, g = make_ctx(dtype, [0] + list(range(13, S)), [0] + [1] * 8, [0, 1, 9], [1, S], [[3, -1, -1], [1, 6, 0]],
                      [3 * page] + [[1, 6, 0][p // page] * page + p % page for p in range(13, S)], page)
    res2 = torch.zeros(9, h, device=DEV)
    att.forward(ctx, torch.cat([other, xn[13:]]).contiguous(), res2, LayerCache(kv=cache, group=g))
    got = torch.cat([res1, res2[1:]]).double().cpu()
    assert (got - ref).abs().max().item() <= tol * ref.abs().max().item()
    assert (res2[:1].double().cpu() - ref_fn(other.double().cpu())).abs().max().item() <= tol * ref.abs().max().item()


# ------------------------------------------------------------------ toy parts, defined in the test
def _register_toys():
    from reinfer_b200.parts.base import FeedForward, Mixer, PositionEncoding, SlotStateSpec, register_part
    from reinfer_b200.weights.params import ParamSpec

    class DecayMixer(Mixer):
        """state <- decay * state + W_in x;  out = W_out state.  The state (one vector per request)
        lives in the cache manager's slots and is carried across steps and portions."""

        def __init__(self, hidden, width, decay):
            self.hidden, self.width, self.decay = hidden, width, decay

        def param_specs(self):
            return {"in.weight": ParamSpec((self.width, self.hidden)), "out.weight": ParamSpec((self.hidden, self.width))}

        def bind(self, t):
            self.w_in, self.w_out = t["in.weight"], t["out.weight"]

        def state_spec(self):
            return SlotStateSpec((self.width,), "float32")

        def forward(self, ctx, xn, residual, cache):
            u = xn.float() @ self.w_in.float().t()
            out = torch.empty_like(u)
            for e in range(ctx.n_entries):
                s = cache.state[ctx.slots[e]]
                for t in range(ctx.q_start[e], ctx.q_start[e + 1]):
                    s.mul_(self.decay).add_(u[t])
                    out[t] = s
            residual += out @ self.w_out.float().t()

    class RoutedFFN(FeedForward):
        """Each token goes to the one expert its router logit picks (router in float32)."""

        def __init__(self, hidden, inter, experts):
            self.hidden, self.inter, self.experts = hidden, inter, experts

        def param_specs(self):
            p = {"router.weight": ParamSpec((self.experts, self.hidden), std=1.0)}
            for i in range(self.experts):
                p[f"experts.{i}.up.weight"] = ParamSpec((self.inter, self.hidden))
                p[f"experts.{i}.down.weight"] = ParamSpec((self.hidden, self.inter))
            return p

        def bind(self, t):
            self.t = t

        def forward(self, ctx, xn, residual):
            choice = (xn.float() @ self.t["router.weight"].float().t()).argmax(-1)
            for i in range(self.experts):
                idx = (choice == i).nonzero().flatten()
                if idx.numel():
                    hdn = torch.relu(xn[idx].float() @ self.t[f"experts.{i}.up.weight"].float().t())
                    residual[idx] += hdn @ self.t[f"experts.{i}.down.weight"].float().t()

    class SignFlip(PositionEncoding):
        """Not a rotation: q and k of odd positions change sign in their first half."""

        def __init__(self, head_dim):
            self.head_dim = head_dim

        def prepare(self, device):
            pass

        def fused_rotary(self):
            return None

        def apply(self, ctx, q, k, positions):
            sign = (1 - 2 * (positions % 2)).to(q.dtype)[:, None, None]
            half = self.head_dim // 2
            q[..., :half] *= sign
            k[..., :half] *= sign

    register_part("mixer", "toy_decay", DecayMixer)
    register_part("ffn", "toy_routed", RoutedFFN)
    register_part("position", "toy_signflip", SignFlip)


def _toy_spec(cfg):
    from reinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    h = cfg.hidden
    norm = lambda p: PartSpec("rmsnorm", {"width": h, "eps": 1e-5}, p)
    attn = lambda p, pos: PartSpec("attention", {"hidden": h, "q_heads": 4, "kv_heads": 2, "head_dim": 16, "position": pos}, p)
    layers = (
        LayerSpec("l0", mixer=PartSpec("toy_decay", {"hidden": h, "width": 24, "decay": 0.9}, "l0.mix."),
                  ffn=PartSpec("swiglu", {"hidden": h, "intermediate": 48}, "l0.ffn."), mixer_norm=norm("l0.n1."), ffn_norm=norm("l0.n2.")),
        LayerSpec("l1", mixer=attn("l1.att.", {"kind": "toy_signflip", "head_dim": 16}),
                  ffn=PartSpec("toy_routed", {"hidden": h, "inter": 40, "experts": 3}, "l1.ffn."), mixer_norm=norm("l1.n1."), ffn_norm=norm("l1.n2.")),
        # reads the keys and values that l1 stored, stores none itself
        LayerSpec("l2", mixer=attn("l2.att.", {"kind": "toy_signflip", "head_dim": 16}),
                  ffn=PartSpec("swiglu", {"hidden": h, "intermediate": 48}, "l2.ffn."), mixer_norm=norm("l2.n1."), ffn_norm=norm("l2.n2."),
                  cache_from="l1"),
    )
    return ModelSpec(hidden_size=h, vocab_size=cfg.vocab, embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h}, "emb."),
                     layers=layers, final_norm=norm("final."), lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "tied": True}, "head."),
                     order=(0, 1, 2, 0))                       # layer 0 runs twice, each run with a state of its own


class _ToyConfig:
    def __init__(self, hidden=32, vocab=97):
        self.hidden, self.vocab = hidden, vocab

    @classmethod
    def from_dict(cls, d):
        return cls(d["toy_hidden"], d["toy_vocab"])

    def to_dict(self):
        return {"architectures": ["ToyStatefulLM"], "toy_hidden": self.hidden, "toy_vocab": self.vocab}


def test_toy_architecture_registered_built_and_stepped(tmp_path):
    """A mixer with state of its own, a routed feed-forward, a non-rotary position encoding, a layer
    that reads another layer's cache and a layer that runs twice: registered from here, written as
    a model folder, loaded by name, and stepped whole / in portions / token by token / mixed with a
    second request.  All cuts must agree (the state, the cache and the batch are carried right)."""
    from reinfer_b200.config import register_architecture, unregister_architecture
    from reinfer_b200.engine import Engine, StepEntry
    from reinfer_b200.parts.base import unregister_part
    from reinfer_b200.weights import write_random_model
    _register_toys()
    register_architecture("ToyStatefulLM", _ToyConfig, _toy_spec)
    try:
        d = write_random_model(str(tmp_path / "toy"), _ToyConfig(), seed=4, dtype=torch.float32)
        assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["ToyStatefulLM"]
        for dtype in ("float32", "bfloat16"):
            seq = [(7 * i + 3) % 97 for i in range(29)]
            other = [(5 * i + 11) % 97 for i in range(12)]

            def run(steps):
                e = Engine.from_model_dir(d, dtype=dtype, page_size=8, max_tokens=64, max_num_seqs=2)
                assert not e.cuda_graphs and [g.layers for g in e.cache.groups] == [("l1",)]     # the toy mixer reads host tables
                assert sorted(e.storage.layer_state) == ["l0", "l0#1"]
                rows = {}
                done = {}
                for entries in steps:
                    lg = e.step([StepEntry(r, t, list(range(len(t)))) for r, t in entries])
                    k = 0
                    for r, t in entries:
                        for i in range(len(t)):
                            rows[(r, done.get(r, 0) + i)] = lg[k].double().cpu()
                            k += 1
                        done[r] = done.get(r, 0) + len(t)
                for r in done:
                    e.finish(r)
                assert e.cache.free_pages() == e.cache.total_pages()
                return rows
            whole = run([[("a", seq)], [("b", other)]])
            portions = run([[("a", seq[:7])], [("a", seq[7:9])], [("a", seq[9:22])], [("a", seq[22:])], [("b", other)]])
            one_by_one = run([[("a", [t])] for t in seq] + [[("b", other)]])
            mixed = run([[("a", seq[:10])], [("a", seq[10:11]), ("b", other[:5])], [("b", other[5:6]), ("a", seq[11:20])],
                         [("a", seq[20:]), ("b", other[6:])]])
            tol = 1e-4 if dtype == "float32" else 4e-2
            for name, got in (("portions", portions), ("one_by_one", one_by_one), ("mixed", mixed)):
                assert got.keys() == whole.keys()
                for key, row in got.items():
                    err = (row - whole[key]).abs().max().item() / whole[key].abs().max().item()
                    assert err <= tol, f"{dtype} {name} {key}: {err:.2e}"
            # the state really matters: the same token at two positions gives different logits
            assert not torch.allclose(whole[("a", 0)], run([[("a", seq[1:2] + seq[:1])]])[("a", 1)], atol=1e-3)
    finally:
        unregister_architecture("ToyStatefulLM")
        for cat, kind in (("mixer", "toy_decay"), ("ffn", "toy_routed"), ("position", "toy_signflip")):
            unregister_part(cat, kind)


def test_stateful_mixer_that_reads_device_tables_keeps_the_decode_graphs(tmp_path):
    """A mixer with state whose single-token step takes its slots from the device table says so, and decode-only
    steps are then replayed from captured graphs; the rows that pad a batch to its bucket point at a slot that
    belongs to nobody.  Eleven requests (bucket of sixteen: five rows of padding) decode together; the logits are
    those of an engine without graphs."""
    from reinfer_b200.config import register_architecture, unregister_architecture
    from reinfer_b200.engine import Engine, StepEntry
    from reinfer_b200.parts.base import Mixer, SlotStateSpec, register_part, unregister_part
    from reinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    from reinfer_b200.weights import write_random_model
    from reinfer_b200.weights.params import ParamSpec

    class TableDecayMixer(Mixer):
        steps_from_device_tables = True

        def __init__(self, hidden, width, decay):
            self.hidden, self.width, self.decay = hidden, width, decay

        def param_specs(self):
            return {"in.weight": ParamSpec((self.width, self.hidden)), "out.weight": ParamSpec((self.hidden, self.width))}

        def bind(self, t):
            self.w_in, self.w_out = t["in.weight"], t["out.weight"]

        def state_spec(self):
            return SlotStateSpec((self.width,), "float32")

        def forward(self, ctx, xn, residual, cache):
            u = xn.float() @ self.w_in.float().t()
            if ctx.max_q_len == 1:                          # single tokens: everything from the device tables
                slots = ctx.entry_slot.long()
                s = cache.state[slots] * self.decay + u
                cache.state[slots] = s
                out = s
            else:
                out = torch.empty_like(u)
                for e in range(ctx.n_entries):
                    s = cache.state[ctx.slots[e]]
                    for t in range(ctx.q_start[e], ctx.q_start[e + 1]):
                        s.mul_(self.decay).add_(u[t])
                        out[t] = s
            residual += out @ self.w_out.float().t()

    def spec(cfg):
        h = cfg.hidden
        norm = lambda p: PartSpec("rmsnorm", {"width": h, "eps": 1e-5}, p)
        layers = tuple(LayerSpec(f"l{i}", mixer=PartSpec("toy_table_decay", {"hidden": h, "width": 24, "decay": 0.8}, f"l{i}.mix."),
                                 ffn=PartSpec("swiglu", {"hidden": h, "intermediate": 48}, f"l{i}.ffn."),
                                 mixer_norm=norm(f"l{i}.n1."), ffn_norm=norm(f"l{i}.n2.")) for i in range(2))
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab, embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h}, "emb."),
                         layers=layers, final_norm=norm("final."),
                         lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "tied": True}, "head."))

    class Config(_ToyConfig):
        def to_dict(self):
            return {"architectures": ["ToyTableLM"], "toy_hidden": self.hidden, "toy_vocab": self.vocab}

    register_part("mixer", "toy_table_decay", TableDecayMixer)
    register_architecture("ToyTableLM", Config, spec)
    try:
        d = write_random_model(str(tmp_path / "toy"), Config(), seed=6, dtype=torch.float32)
        n = 11
        prompts = {f"r{i}": [(3 * i + 7 * k + 1) % 97 for k in range(2 + i % 4)] for i in range(n)}
        tails = {r: [(5 * i + 11 * k + 2) % 97 for k in range(5)] for i, r in enumerate(prompts)}

        def run(graphs):
            e = Engine.from_model_dir(d, dtype="float32", max_tokens=64, max_num_seqs=n, cuda_graphs=graphs)
            assert e.cuda_graphs == graphs and not e.cache.groups and len(e.storage.layer_state) == 2
            rows = [e.step([StepEntry(r, p, [len(p) - 1]) for r, p in prompts.items()])]
            for k in range(5):
                live = [r for i, r in enumerate(prompts) if not (k >= 3 and i % 3 == 0)]      # some leave early
                rows.append(e.step([StepEntry(r, [tails[r][k]], [0]) for r in live]))
                if k == 2:
                    for i, r in enumerate(prompts):
                        if i % 3 == 0:
                            e.finish(r)
            return torch.cat(rows).double().cpu(), e.graph_replays
        eager, n0 = run(False)
        graphed, n1 = run(True)
        assert n0 == 0 and n1 == 5
        assert (graphed - eager).abs().max().item() <= 1e-5 * eager.abs().max().item()
    finally:
        unregister_architecture("ToyTableLM")
        unregister_part("mixer", "toy_table_decay")


def test_a_block_with_four_norms_needs_a_block_class_only(tmp_path):
    """A layer is a block over parts named by role, and which roles there are is the block's business: a
    'sandwich' arrangement (a norm before and a norm after the mixer, and the same around the feed-forward) is
    defined and registered here, built from a model folder and stepped under several cuts, and agrees with the
    same arithmetic written with the plain functions."""
    from reinfer_b200.config import register_architecture, unregister_architecture
    from reinfer_b200.engine import Engine, StepEntry
    from reinfer_b200.parts.base import register_part, unregister_part
    from reinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    from reinfer_b200.weights import write_random_model

    class SandwichBlock:
        roles = ("pre_mixer_norm", "mixer", "post_mixer_norm", "pre_ffn_norm", "ffn", "post_ffn_norm")

        def __init__(self, parts):
            assert set(self.roles) <= set(parts)
            self.p = parts

        def forward(self, ctx, x, cache):
            p = self.p
            for pre, inner, post, args in ((p["pre_mixer_norm"], p["mixer"], p["post_mixer_norm"], (cache,)),
                                           (p["pre_ffn_norm"], p["ffn"], p["post_ffn_norm"], ())):
                branch = torch.zeros_like(x)                        # the inner part adds its output into what it is given
                inner.forward(ctx, pre.forward(ctx, x), branch, *args)
                x += post.forward(ctx, branch).float()

    H, V, QH, KH, D, F = 48, 101, 4, 2, 16, 80

    def spec(cfg):
        norm = lambda p, eps=1e-5: PartSpec("rmsnorm", {"width": H, "eps": eps}, p)
        layers = tuple(LayerSpec(
            f"l{i}", block="toy_sandwich",
            pre_mixer_norm=norm(f"l{i}.n1."), post_mixer_norm=norm(f"l{i}.n2."),
            mixer=PartSpec("attention", {"hidden": H, "q_heads": QH, "kv_heads": KH, "head_dim": D, "qk_norm": True,
                                         "qk_norm_eps": 1e-5, "position": {"kind": "rope", "head_dim": D, "theta": 1e4}},
                           f"l{i}.att."),
            pre_ffn_norm=norm(f"l{i}.n3."), post_ffn_norm=norm(f"l{i}.n4."),
            ffn=PartSpec("swiglu", {"hidden": H, "intermediate": F}, f"l{i}.ffn.")) for i in range(2))
        return ModelSpec(hidden_size=H, vocab_size=V, embedding=PartSpec("embedding", {"vocab": V, "hidden": H}, "emb."),
                         layers=layers, final_norm=norm("final."),
                         lm_head=PartSpec("linear", {"vocab": V, "hidden": H, "tied": True}, "head."))

    class Config(_ToyConfig):
        def to_dict(self):
            return {"architectures": ["ToySandwichLM"], "toy_hidden": H, "toy_vocab": V}

    def plain_forward(w, tokens):
        cfg = dict(num_attention_heads=QH, num_key_value_heads=KH, head_dim=D, rms_norm_eps=1e-5, rope_theta=1e4, hidden_size=H)
        pos = torch.arange(len(tokens))
        x = plain.embed(w["emb.weight"], tokens)
        for i in range(2):
            a = plain.attention_block(plain.rms_norm(x, w[f"l{i}.n1.weight"], 1e-5), w, f"l{i}.att.", cfg, pos)
            x = x + plain.rms_norm(a, w[f"l{i}.n2.weight"], 1e-5)
            f = plain.swiglu_ffn(plain.rms_norm(x, w[f"l{i}.n3.weight"], 1e-5), w[f"l{i}.ffn.gate_proj.weight"],
                                 w[f"l{i}.ffn.up_proj.weight"], w[f"l{i}.ffn.down_proj.weight"])
            x = x + plain.rms_norm(f, w[f"l{i}.n4.weight"], 1e-5)
        return plain.linear(plain.rms_norm(x, w["final.weight"], 1e-5), w["emb.weight"])

    register_part("block", "toy_sandwich", SandwichBlock)
    register_architecture("ToySandwichLM", Config, spec)
    try:
        d = write_random_model(str(tmp_path / "toy"), Config(), seed=8, dtype=torch.float32)
        w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
        seq = [(13 * i + 2) % V for i in range(37)]
        ref = plain_forward(w, seq)
        for cuts in ([37], [9, 2, 17, 1, 1, 7], [1] * 37):
            e = Engine.from_model_dir(d, dtype="float32", page_size=8, max_tokens=40, max_num_seqs=1)
            rows, i = [], 0
            for n in cuts:
                rows.append(e.step([StepEntry("a", seq[i:i + n], list(range(n)))]).double().cpu())
                i += n
            got = torch.cat(rows)
            assert (got - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
        # a layer that lacks a role its block needs is refused when the model is built, by name
        with pytest.raises(ValueError, match="ffn_norm"):
            from reinfer_b200.parts.model import Model
            Model(ModelSpec(hidden_size=H, vocab_size=V, embedding=PartSpec("embedding", {"vocab": V, "hidden": H}, "emb."),
                            layers=(LayerSpec("l0", block="prenorm", mixer=spec(None).layers[0].mixer,
                                              ffn=spec(None).layers[0].ffn, mixer_norm=spec(None).layers[0].pre_mixer_norm),),
                            final_norm=PartSpec("rmsnorm", {"width": H, "eps": 1e-5}, "final."),
                            lm_head=PartSpec("linear", {"vocab": V, "hidden": H, "tied": True}, "head.")))
    finally:
        unregister_architecture("ToySandwichLM")
        unregister_part("block", "toy_sandwich")


def _window_spec(cfg):
    """Two attention layers that see every key and one that sees only the last 24: two cache groups."""
    from reinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
    h = cfg.hidden
    norm = lambda p: PartSpec("rmsnorm", {"width": h, "eps": 1e-5}, p)

    def attn(p, window):
        return PartSpec("attention", {"hidden": h, "q_heads": 4, "kv_heads": 2, "head_dim": 16, "qk_norm": True,
                                      "qk_norm_eps": 1e-5, "window": window,
                                      "position": {"kind": "rope", "head_dim": 16, "theta": 1e4}}, p)
    ffn = lambda p: PartSpec("swiglu", {"hidden": h, "intermediate": 48}, p)
    layers = tuple(LayerSpec(f"l{i}", mixer=attn(f"l{i}.att.", w), ffn=ffn(f"l{i}.ffn."), mixer_norm=norm(f"l{i}.n1."),
                             ffn_norm=norm(f"l{i}.n2.")) for i, w in enumerate([None, 24, None]))
    return ModelSpec(hidden_size=h, vocab_size=cfg.vocab, embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": h}, "emb."),
                     layers=layers, final_norm=norm("final."), lm_head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": h, "tied": True}, "head."))


class _WinConfig(_ToyConfig):
    def to_dict(self):
        return {"architectures": ["ToyWindowLM"], "toy_hidden": self.hidden, "toy_vocab": self.vocab}


@pytest.mark.parametrize("dtype,page", [("float32", 8), ("bfloat16", 8), ("bfloat16", 4)])
def test_window_group_gives_pages_back_and_all_cuts_agree(tmp_path, dtype, page):
    """A layer with a window lives in a cache group of its own; its pages go back to the pool as the
    window passes them, the kernels never touch a page that was given back, and whole / portions /
    token-by-token give the same logits (the window's edge at every kind of step boundary)."""
    from reinfer_b200.config import register_architecture, unregister_architecture
    from reinfer_b200.engine import Engine, StepEntry
    from reinfer_b200.weights import write_random_model
    register_architecture("ToyWindowLM", _WinConfig, _window_spec)
    try:
        d = write_random_model(str(tmp_path / "win"), _WinConfig(), seed=9, dtype=torch.float32)
        seq = [(11 * i + 5) % 97 for i in range(150)]

        def run(cuts):
            e = Engine.from_model_dir(d, dtype=dtype, page_size=page, max_tokens=192, max_num_seqs=2)
            assert [g.window for g in e.cache.groups] == [None, 24] and [g.layers for g in e.cache.groups] == [("l0", "l2"), ("l1",)]
            # poison the pools: a read of a page that is not held would show
            for arr in e.storage.group_arrays:
                arr.fill_(float("nan"))
            rows, i = [], 0
            for n in cuts:
                lg = e.step([StepEntry("a", seq[i:i + n], list(range(n)))])
                rows.append(lg.double().cpu())
                i += n
                e.cache.check()
                held = sum(1 for p in e.cache.table("a", 1) if p >= 0)
                assert held <= -(-24 // page) + 1 + -(-n // page)            # the window's pages (+ this step's)
            assert i == len(seq)
            assert sum(1 for p in e.cache.table("a", 0) if p >= 0) == -(-len(seq) // page)
            e.finish("a")
            assert all(g.pool.in_use == 0 for g in e.cache.groups)
            return torch.cat(rows)
        whole = run([150])
        assert not torch.isnan(whole).any()
        tol = 1e-4 if dtype == "float32" else 4e-2
        for cuts in ([23, 1, 1, 25, 2, 48, 50], [1] * 150, [100] + [1] * 50, [7] * 21 + [3]):
            got = run(cuts)
            err = ((got - whole).abs().max(dim=1).values / whole.abs().max(dim=1).values).max().item()
            assert err <= tol, f"{dtype} cuts {cuts[:4]}..: {err:.2e}"
        # the window matters: with every key visible the late logits differ
        assert (whole[100:] - whole[100:].mean()).abs().max() > 0
    finally:
        unregister_architecture("ToyWindowLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotary_part_unfused_apply(dtype):
    """RotaryEncoding.apply (the form a foreign mixer would call) against the plain rotation, partial width too."""
    from reinfer_b200.parts.rope import RotaryEncoding
    for d, rot in ((32, 32), (48, 16)):
        r = RotaryEncoding(head_dim=d, theta=1e4, rotary_dim=rot)
        r.prepare(DEV)
        pos = torch.tensor([0, 3, 77, 1000], dtype=torch.int32, device=DEV)
        q, k = torch.randn(4, 5, d, device=DEV).to(dtype), torch.randn(4, 2, d, device=DEV).to(dtype)
        q0, k0 = q.clone(), k.clone()
        ctx, _ = make_ctx(dtype, pos.tolist(), [0] * 4, [0, 4], [1001])
        r.apply(ctx, q, k, pos)
        for got, src in ((q, q0), (k, k0)):
            ref = torch.cat([plain.rope_half_split(src[..., :rot].double().cpu(), pos.cpu(), 1e4), src[..., rot:].double().cpu()], -1)
            # the angle is a float32 product: at position 1000 it is off by up to 6e-5 rad from the float64 angle
            tol = 2e-2 if dtype == torch.bfloat16 else 5e-5
            assert (got.double().cpu() - ref).abs().max().item() <= tol * ref.abs().max().item()
