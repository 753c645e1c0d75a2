"""What another architecture can be made of without a change to the package's files: a block
arrangement with slots of its own (one norm, two mixers side by side, an optional feed-forward),
a scaled embedding with a learned table of absolute positions, scaled and capped logits, two
attention layers that agree in head counts and differ in head size, and a mixer with per-request
state that decodes under CUDA graphs.  Toy parts only, defined here; none is anybody's model."""

from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain
from conftest import random_tokens

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- toy parts
@dataclass(frozen=True)
class CarrySpec:
    """y_t = s_t, s_t = decay * s_{t-1} + x_t @ W^T, s kept per request in a state row (hidden floats)."""

    family = "mixer"
    kind: str = "toy_carry"
    prefix: str = ""
    hidden_size: int = 0
    decay: float = 0.5


class CarryMixer:
    """State on the device, indexed by the context's device arrays only, so that a decode step can
    be captured in a CUDA graph and replayed.  Portions of several tokens run token by token."""

    capturable = True

    @staticmethod
    def params(spec):
        from tandem_b200.config.plan import ParamSpec, WeightSource

        return {"w": ParamSpec((spec.hidden_size, spec.hidden_size), (WeightSource(f"{spec.prefix}.w"),))}

    @staticmethod
    def kv_need(spec):
        return None

    @staticmethod
    def state_need(spec):
        from tandem_b200.parts.base import StateNeed

        return StateNeed((spec.hidden_size,), torch.float32)

    def __init__(self, spec, weights, dtype, device):
        self.spec, self.w = spec, weights["w"]

    def forward(self, x, ctx):
        state = ctx.state(self)  # two mixers share a layer here: each names itself
        u = x.float() @ self.w.float().T
        slots = ctx.state_slots.long()
        if ctx.max_new == 1:  # one token per request: nothing but device-side indexing
            s = self.spec.decay * state.index_select(0, slots) + u
            state.index_copy_(0, slots, s)
            return s.to(x.dtype)
        out = torch.empty_like(u)
        at = 0
        for b, n in enumerate(ctx.host_lens):
            s = state[slots[b]]
            for t in range(at, at + n):
                s = self.spec.decay * s + u[t]
                out[t] = s
            state[slots[b]] = s
            at += n
        return out.to(x.dtype)


class SideBySide:
    """One norm; attention and the carry mixer read the same normalised rows and their outputs
    are added; a feed-forward may join them."""

    slots = {"norm": "norm", "attention": "mixer", "carry": "mixer"}
    optional_slots = {"feed_forward": "feed_forward"}

    def forward(self, layer, x, residual, ctx):
        h = layer.norm.forward(x, residual, ctx.dtype)
        out = layer.attention.forward(h, ctx) + layer.carry.forward(h, ctx)
        if "feed_forward" in layer.parts:
            out = out + layer.feed_forward.forward(h, ctx)
        return out


def register():
    from tandem_b200.registry import register_part

    register_part("mixer", "toy_carry", CarryMixer)
    register_part("block", "toy_side_by_side", SideBySide)


def attention_spec(prefix, H, nh, nkv, hd, theta=100.0):
    from tandem_b200.config.plan import AttentionSpec, PositionSpec

    return AttentionSpec("attention", prefix=prefix, hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                         scale=hd ** -0.5, qk_norm=False, position=PositionSpec("rope", rotary_dim=hd, theta=theta, max_position=256))


def attention_weights(g, prefix, H, nh, nkv, hd, s=0.2):
    return {f"{prefix}.q_proj.weight": torch.randn(nh * hd, H, generator=g) * s, f"{prefix}.k_proj.weight": torch.randn(nkv * hd, H, generator=g) * s,
            f"{prefix}.v_proj.weight": torch.randn(nkv * hd, H, generator=g) * s, f"{prefix}.o_proj.weight": torch.randn(H, nh * hd, generator=g) * s}


def plain_attention(x, w, prefix, nh, nkv, hd, theta):
    """Whole-sequence attention without q/k norms, in the dtype of x."""
    T = x.shape[0]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(T, nh, hd)
    k = (x @ w[f"{prefix}.k_proj.weight"].T).view(T, nkv, hd)
    v = (x @ w[f"{prefix}.v_proj.weight"].T).view(T, nkv, hd)
    cos, sin = plain.rope_tables(hd, theta, T, x.dtype)
    q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
    return plain.attention_scores(q, k, v, None).reshape(T, nh * hd) @ w[f"{prefix}.o_proj.weight"].T


def plain_carry(x, w, decay):
    u = x @ w.T
    out, s = torch.empty_like(u), torch.zeros_like(u[0])
    for t in range(x.shape[0]):
        s = decay * s + u[t]
        out[t] = s
    return out


def side_by_side_model(dtype, H=48, V=70, nh=4, nkv=2, hd=16):
    """Layer 0: the toy arrangement with a feed-forward; layer 1: without; layer 2: the package's
    pre-norm layer.  Embedding scaled and with learned positions; logits scaled and capped."""
    from tandem_b200.config.plan import EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelPlan, NormSpec, RunStep
    from tandem_b200.models.decoder import Decoder
    from tandem_b200.weights.loader import TensorDict

    register()
    layers = []
    for i in range(2):
        slots = dict(norm=NormSpec("rmsnorm", H, 1e-5, f"l{i}.n"), attention=attention_spec(f"l{i}.attn", H, nh, nkv, hd),
                     carry=CarrySpec(prefix=f"l{i}.carry", hidden_size=H, decay=0.6 + 0.2 * i))
        if i == 0:
            slots["feed_forward"] = GatedMLPSpec("gated_mlp", "l0.mlp", H, 2 * H)
        layers.append(LayerSpec.of("toy_side_by_side", **slots))
    layers.append(LayerSpec.of("prenorm", mixer=attention_spec("l2.attn", H, nh, nkv, hd), feed_forward=GatedMLPSpec("gated_mlp", "l2.mlp", H, 2 * H),
                               mixer_norm=NormSpec("rmsnorm", H, 1e-5, "l2.n1"), feed_forward_norm=NormSpec("rmsnorm", H, 1e-5, "l2.n2")))
    plan = ModelPlan(embedding=EmbeddingSpec(V, H, "emb", scale=H ** 0.5, positions="pos"), layers=tuple(layers),
                     order=tuple(RunStep(i) for i in range(3)), final_norm=NormSpec("rmsnorm", H, 1e-5, "fn"),
                     head=HeadSpec(V, H, "head", scale=0.5, softcap=2.5), max_position=256)
    g = torch.Generator().manual_seed(12)
    w = {"emb": torch.randn(V, H, generator=g) * 0.1, "pos": torch.randn(256, H, generator=g) * 0.3, "fn": torch.ones(H),
         "head": torch.randn(V, H, generator=g) * 0.3}
    for i in range(3):
        w.update(attention_weights(g, f"l{i}.attn", H, nh, nkv, hd))
    for i in range(2):
        w[f"l{i}.n"] = 1 + 0.1 * torch.randn(H, generator=g)
        w[f"l{i}.carry.w"] = torch.randn(H, H, generator=g) * 0.1
    w["l2.n1"], w["l2.n2"] = 1 + 0.1 * torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
    for p in ("l0.mlp", "l2.mlp"):
        w.update({f"{p}.gate_proj.weight": torch.randn(2 * H, H, generator=g) * 0.1, f"{p}.up_proj.weight": torch.randn(2 * H, H, generator=g) * 0.1,
                  f"{p}.down_proj.weight": torch.randn(H, 2 * H, generator=g) * 0.1})
    w = {k: v.bfloat16().float() for k, v in w.items()}  # the same numbers in both dtypes
    decoder = Decoder(plan, TensorDict(dict(w)), dtype, "cuda")
    return decoder, w, dict(H=H, V=V, nh=nh, nkv=nkv, hd=hd)


def side_by_side_plain(w, d, tokens):
    """The same model in float64, whole sequence, straight from its formulas."""
    w = {k: v.double() for k, v in w.items()}
    ids = torch.tensor(tokens)
    h = d["H"] ** 0.5 * w["emb"][ids] + w["pos"][: len(ids)]
    for i in range(2):
        x = plain.rms_norm(h, w[f"l{i}.n"], 1e-5)
        out = plain_attention(x, w, f"l{i}.attn", d["nh"], d["nkv"], d["hd"], 100.0) + plain_carry(x, w[f"l{i}.carry.w"], 0.6 + 0.2 * i)
        if i == 0:
            out = out + plain.swiglu(x, w, "l0.mlp")
        h = h + out
    h = h + plain_attention(plain.rms_norm(h, w["l2.n1"], 1e-5), w, "l2.attn", d["nh"], d["nkv"], d["hd"], 100.0)
    h = h + plain.swiglu(plain.rms_norm(h, w["l2.n2"], 1e-5), w, "l2.mlp")
    logits = 0.5 * (plain.rms_norm(h, w["fn"], 1e-5) @ w["head"].T)
    return 2.5 * torch.tanh(logits / 2.5)


# ----------------------------------------------------------------------------- tests
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_an_arrangement_with_slots_of_its_own_and_embedding_and_head_hooks(dtype):
    from tandem_b200.engine.core import build_executor
    from tandem_b200.engine.executor import StepEntry

    decoder, w, d = side_by_side_model(dtype)
    assert decoder.cache_users == [(0, "attention"), (0, "carry"), (1, "attention"), (1, "carry"), (2, "mixer")]
    assert [n is not None for n in decoder.kv_needs()] == [True, False, True, False, True]
    assert [n is not None for n in decoder.state_needs()] == [False, True, False, True, False]
    ex = build_executor(decoder, page_size=8, num_pages=24, max_requests=3)
    a, b = random_tokens(31, 45, d["V"]), random_tokens(32, 26, d["V"])
    whole_a = ex.step([StepEntry("a", a, list(range(45)))], end=["a"])
    whole_b = ex.step([StepEntry("b", b, list(range(26)))], end=["b"])
    got_a, got_b, ia, ib = [], [], 0, 0
    for na, nb in ((9, 2), (2, 7), (33, 1), (1, 16)):  # portions of one beside single tokens of the other
        out = ex.step([StepEntry("a2", a[ia: ia + na], list(range(na))), StepEntry("b2", b[ib: ib + nb], list(range(nb)))])
        got_a.append(out[:na]), got_b.append(out[na:])
        ia, ib = ia + na, ib + nb
    ex.step([], end=["a2", "b2"])
    assert ex.manager.all_free()
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.06, rtol=0.05)
    torch.testing.assert_close(torch.cat(got_a), whole_a, **tol)
    torch.testing.assert_close(torch.cat(got_b), whole_b, **tol)
    for tokens, got in ((a, whole_a), (b, whole_b)):
        want = side_by_side_plain(w, d, tokens)
        assert want.abs().max() > 1.0  # the cap bends the logits: it is not a no-op here
        torch.testing.assert_close(got.cpu().double(), want, **(dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else tol))


def test_a_layer_that_lacks_a_slot_or_brings_an_unknown_one_is_refused():
    from tandem_b200.config.model_config import ConfigError
    from tandem_b200.config.plan import EmbeddingSpec, HeadSpec, LayerSpec, ModelPlan, NormSpec, RunStep
    from tandem_b200.models.decoder import Decoder
    from tandem_b200.weights.loader import TensorDict

    register()
    H = 32
    bad = LayerSpec.of("toy_side_by_side", norm=NormSpec("rmsnorm", H, 1e-5, "n"), attention=attention_spec("a", H, 2, 1, 16),
                       extra_norm=NormSpec("rmsnorm", H, 1e-5, "n2"))
    plan = ModelPlan(embedding=EmbeddingSpec(10, H, "emb"), layers=(bad,), order=(RunStep(0),),
                     final_norm=NormSpec("rmsnorm", H, 1e-5, "fn"), head=HeadSpec(10, H, None), max_position=64)
    with pytest.raises(ConfigError, match=r"missing \['carry'\], unknown \['extra_norm'\]"):
        Decoder(plan, TensorDict({}), torch.float32, "cuda")


def test_two_attention_layers_with_equal_head_counts_and_other_head_sizes():
    """Head sizes 64 and 40 under the same (window, heads, kv heads): the first runs the tensor-core
    kernels, the second, whose head size they do not take, the CUDA-core kernel; each layer has to
    get its own plan."""
    from tandem_b200.config.plan import EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelPlan, NormSpec, RunStep
    from tandem_b200.engine.core import build_executor
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.kernels import attention as attention_kernels
    from tandem_b200.models.decoder import Decoder
    from tandem_b200.weights.loader import TensorDict

    H, V, nh, nkv = 64, 80, 4, 2
    sizes = (64, 40)
    assert attention_kernels.tensor_core_path_applies(torch.bfloat16, 64, 16, 2)
    assert not attention_kernels.tensor_core_path_applies(torch.bfloat16, 40, 16, 2)
    layers = tuple(LayerSpec.of("prenorm", mixer=attention_spec(f"l{i}.attn", H, nh, nkv, hd), feed_forward=GatedMLPSpec("gated_mlp", f"l{i}.mlp", H, 2 * H),
                                mixer_norm=NormSpec("rmsnorm", H, 1e-5, f"l{i}.n1"), feed_forward_norm=NormSpec("rmsnorm", H, 1e-5, f"l{i}.n2"))
                   for i, hd in enumerate(sizes))
    plan = ModelPlan(embedding=EmbeddingSpec(V, H, "emb"), layers=layers, order=(RunStep(0), RunStep(1)),
                     final_norm=NormSpec("rmsnorm", H, 1e-5, "fn"), head=HeadSpec(V, H, None), max_position=256)
    g = torch.Generator().manual_seed(4)
    w = {"emb": torch.randn(V, H, generator=g) * 0.5, "fn": torch.ones(H)}
    for i, hd in enumerate(sizes):
        w.update(attention_weights(g, f"l{i}.attn", H, nh, nkv, hd))
        w.update({f"l{i}.n1": 1 + 0.1 * torch.randn(H, generator=g), f"l{i}.n2": torch.ones(H),
                  f"l{i}.mlp.gate_proj.weight": torch.randn(2 * H, H, generator=g) * 0.1,
                  f"l{i}.mlp.up_proj.weight": torch.randn(2 * H, H, generator=g) * 0.1,
                  f"l{i}.mlp.down_proj.weight": torch.randn(H, 2 * H, generator=g) * 0.1})
    w = {k: v.bfloat16().float() for k, v in w.items()}
    decoder = Decoder(plan, TensorDict(dict(w)), torch.bfloat16, "cuda")
    ex = build_executor(decoder, page_size=16, num_pages=16, max_requests=3)
    assert len(ex.manager.groups) == 2  # one pool per head size
    tokens = random_tokens(8, 90, V)
    whole = ex.step([StepEntry("w", tokens, list(range(90)))], end=["w"])
    got, at = [], 0
    for n in (40, 2, 30, 1, 1, 16):
        got.append(ex.step([StepEntry("p", tokens[at: at + n], list(range(n)))]))
        at += n
    ex.step([], end=["p"])
    def run_plain(dtype):
        wd = {k: v.to(dtype) for k, v in w.items()}
        h = wd["emb"][torch.tensor(tokens)]
        for i, hd in enumerate(sizes):
            h = h + plain_attention(plain.rms_norm(h, wd[f"l{i}.n1"], 1e-5), wd, f"l{i}.attn", nh, nkv, hd, 100.0)
            h = h + plain.swiglu(plain.rms_norm(h, wd[f"l{i}.n2"], 1e-5), wd, f"l{i}.mlp")
        return (plain.rms_norm(h, wd["fn"], 1e-5) @ wd["emb"].T).double()

    want = run_plain(torch.float64)
    base = (run_plain(torch.bfloat16) - want).abs().max().item()  # what plain bfloat16 arithmetic loses on this model
    for got_logits in (whole, torch.cat(got)):
        err = (got_logits.cpu().double() - want).abs().max().item()
        assert err <= 1.5 * base + 0.02, (err, base)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_mixer_with_state_decodes_under_cuda_graphs(dtype):
    """Three requests decode through the graph of four rows: the padding row's state goes to the row
    of no request, so the request that holds state row 0 is not disturbed; the logits are the
    eager step function's and the plain float64 model's."""
    from tandem_b200.engine.core import build_executor
    from tandem_b200.engine.cuda_graph import DecodeGraphs
    from tandem_b200.engine.executor import StepEntry

    decoder, w, d = side_by_side_model(dtype)
    graph = build_executor(decoder, page_size=8, num_pages=32, max_requests=4)
    eager = build_executor(decoder, page_size=8, num_pages=32, max_requests=4)
    graphs = DecodeGraphs.maybe(graph, 4, 128)
    assert graphs is not None  # per-request state no longer keeps a model away from graphs
    toks = {f"r{i}": random_tokens(60 + i, n, d["V"]) for i, n in enumerate((30, 21, 44))}
    head = {"r0": 12, "r1": 3, "r2": 25}
    for ex in (graph, eager):
        ex.step([StepEntry(rid, t[: head[rid]], []) for rid, t in toks.items()])
    assert graph.manager.slot("r0") == 0
    at = dict(head)
    got = {rid: {} for rid in toks}
    for _ in range(19):
        live = [rid for rid in toks if at[rid] < len(toks[rid])]
        entries = [StepEntry(rid, [toks[rid][at[rid]]], [0]) for rid in live]
        assert graphs.takes(entries)
        for ex in (graph, eager):
            for e in entries:
                assert ex.manager.grow(e.request_id, at[e.request_id] + 1)
        a = graphs.run(entries).clone()
        b = eager.run(entries)
        for ex in (graph, eager):
            for e in entries:
                ex.manager.commit(e.request_id, 1)
        if dtype == torch.float32:
            assert torch.equal(a, b)
        else:
            torch.testing.assert_close(a, b, atol=0.05, rtol=0.05)
        for row, rid in zip(a.double().cpu(), live):
            got[rid][at[rid]] = row
            at[rid] += 1
    assert set(graphs.captured) >= {4, 1} and all(c.launches > 0 for c in graphs.captured.values())
    # steps with prompt portions are captured only for mixers that say they read such a batch from the device
    # alone; the toy mixer walks the requests on the host, so a model that has it keeps those steps eager
    assert not graphs.mixed and not graphs.takes([StepEntry("r0", [1, 2, 3], [2])])
    if dtype == torch.bfloat16:
        wide_heads, _, _ = side_by_side_model(dtype, hd=64)  # a head size with which the attention layers alone would qualify
        assert not DecodeGraphs.maybe(build_executor(wide_heads, page_size=16, num_pages=8, max_requests=4), 4, 128).mixed
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=0.06, rtol=0.05)
    for rid, rows in got.items():
        want = side_by_side_plain(w, d, toks[rid])
        for pos, row in rows.items():
            torch.testing.assert_close(row, want[pos], **tol)
