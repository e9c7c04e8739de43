"""Each part alone against the plain model's function, and the generality of the assembly:
a toy mixer with state of its own, a toy architecture with a window in some layers, a layer
that runs twice and a layer that reads another layer's cache - all registered from here,
without a change to the framework's files."""
import math

import pytest
import torch

import plain_model as pm
import trace_util as tu
from gpu_util import TOL

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig
from tiny_transformer_inference_engine_b200 import register_model, register_part
from tiny_transformer_inference_engine_b200.parts.base import (PartSpec, LayerSpec, RunEntry, ModelSpec, Mixer, ParamSpec,
                                                                FeedForward, PositionEncoding, FixedStateNeed, StepContext,
                                                                PagedKVView)
from tiny_transformer_inference_engine_b200.registry import build_part, unregister_model, unregister_part
from tiny_transformer_inference_engine_b200.weights import random_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    return get_ops(DEV)


def rel(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max()).item()


def ctx_for(ops, dtype, seqs, page, tables):
    """A StepContext for requests given as (start, new tokens)."""
    pos = [s + i for s, n in seqs for i in range(n)]
    tseq = [i for i, (_, n) in enumerate(seqs) for _ in range(n)]
    qsl = [0]
    for _, n in seqs:
        qsl.append(qsl[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(ops=ops, dtype=dtype, device=torch.device(DEV), num_tokens=len(pos), num_seqs=len(seqs),
                       max_q_len=max(n for _, n in seqs), max_kv_len=max(s + n for s, n in seqs), token_ids=t([0] * len(pos)),
                       positions=t(pos), token_seq=t(tseq), query_start_loc=t(qsl), seq_lens=t([s + n for s, n in seqs]),
                       slot_ids=t(list(range(len(seqs)))), logit_rows=t([0]), num_logit_rows=0, block_tables={0: tables})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(ops, dtype):
    part = build_part("norm", PartSpec("rmsnorm", "n", {"dim": 200, "eps": 3e-4}))
    part.bind(ops, DT[dtype], torch.device(DEV))
    w = 1 + 0.2 * torch.randn(200)
    part.load({"weight": w.to(DEV)})
    resid, delta = torch.randn(7, 200), torch.randn(7, 200).to(DT[dtype])
    r = resid.clone().to(DEV)
    out = part.add_norm(r, delta.to(DEV))
    x = resid + delta.float()
    assert rel(r.cpu(), x) < 1e-6
    assert rel(out.float().cpu(), pm.plain_rmsnorm(x, w, 3e-4)) < (1e-5 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ffn_part(ops, dtype):
    part = build_part("ffn", PartSpec("swiglu", "mlp", {"d_model": 72, "hidden": 200, "bias": True}))
    part.bind(ops, DT[dtype], torch.device(DEV))
    g = torch.Generator().manual_seed(0)
    w = {k: (torch.randn(ps.shape, generator=g) * 0.1).to(DT[dtype]) for k, ps in part.param_specs().items()}
    part.load({k: v.to(DEV) for k, v in w.items()})
    x = torch.randn(9, 72, generator=g).to(DT[dtype])
    out = part.forward(x.to(DEV), None)
    exp = pm.plain_swiglu(x.float(), {f"mlp.{k}": v.float() for k, v in w.items()}, "mlp")
    assert rel(out.float().cpu(), exp) < (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("style", ["interleaved", "half"])
def test_attention_part_with_position_encoding(ops, dtype, style):
    """The mixer alone: a whole sequence in one step, then the same in two portions from the cache."""
    d, Hq, Hkv, D, page, S = 96, 6, 2, 16, 4, 23
    cfg = {"d_model": d, "num_heads": Hq, "num_kv_heads": Hkv, "rope_theta": 777.0}
    part = build_part("mixer", PartSpec("attention", "attn", {
        "d_model": d, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "bias": True,
        "position": PartSpec("rope", "", {"dim": D, "base": 777.0, "style": style})}))
    part.bind(ops, DT[dtype], torch.device(DEV))
    g = torch.Generator().manual_seed(1)
    w = {k: (torch.randn(ps.shape, generator=g) * 0.1).to(DT[dtype]) for k, ps in part.param_specs().items()}
    part.load({k: v.to(DEV) for k, v in w.items()})
    x = torch.randn(S, d, generator=g).to(DT[dtype])
    exp = pm.plain_mqa(x.float(), {f"attn.{k}": v.float() for k, v in w.items()}, "attn", cfg, torch.arange(S), style=style)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for cuts in ([S], [10, 13], [1, 2, 20]):
        kp = torch.zeros(8, Hkv, page, D, dtype=DT[dtype], device=DEV)
        vp = torch.zeros_like(kp)
        table = torch.tensor([[5, 2, 7, 1, 3, 6]], dtype=torch.int32, device=DEV)
        outs, start = [], 0
        for n in cuts:
            ctx = ctx_for(ops, DT[dtype], [(start, n)], page, table)
            outs.append(part.forward(x[start:start + n].to(DEV), ctx, PagedKVView(kp, vp, table, page)))
            start += n
        assert rel(torch.cat(outs).float().cpu(), exp) < tol, cuts


# ------------------------------------------------------------------------------------------ toy parts
class ToyDecayMixer(Mixer):
    """A mixer with state of its own and no pages: s_t = a * s_{t-1} + W x_t per request, y_t = s_t.
    Its state lives in the state slot of the request; a portion advances it token by token on the host,
    a step of single tokens advances every request at once on the device (so a decode step can be
    captured: the padding rows of a captured step carry slot -1, which indexes the scratch row)."""

    capturable = "decode"              # a portion is advanced on the host: only steps of single tokens can be captured

    def __init__(self, prefix, dim, decay):
        super().__init__(prefix)
        self.dim, self.decay = dim, decay

    def param_specs(self):
        return {"mix.weight": ParamSpec((self.dim, self.dim))}

    def load(self, params):
        self.w = params["mix.weight"]

    def cache_need(self):
        return FixedStateNeed((self.dim,), "float32")

    def forward(self, x, ctx, cache):
        u = self.ops.linear(x, self.w, None).float()
        if ctx.max_q_len == 1 and self.capturable:
            rows = torch.remainder(ctx.slot_ids.long(), cache.state.shape[0])
            s = self.decay * cache.state[rows] + u
            cache.state.index_copy_(0, rows, s)
            return s.to(x.dtype)
        y = torch.empty_like(u)
        qsl, slots = ctx.host["query_start_loc"], ctx.slot_ids.tolist()
        for i in range(ctx.num_seqs):
            s = cache.state[slots[i]]
            for t in range(qsl[i], qsl[i + 1]):
                s = self.decay * s + u[t]
                y[t] = s
            cache.state[slots[i]] = s
        return y.to(x.dtype)


class ToyHostDecayMixer(ToyDecayMixer):
    """The same, always on the host: a part that reads device values in its step says so, and the engine then
    runs the model without captured graphs."""
    capturable = False


class ToyAttentionPlusDecay(Mixer):
    """A mixer that keeps two things between steps - pages of keys and values, and a state of fixed size - as the
    sum of an attention part and a decay part; it reports both needs and gets both views."""

    def __init__(self, prefix, attention, decay):
        super().__init__(prefix)
        self.attn, self.toy = build_part("mixer", attention), build_part("mixer", decay)

    def children(self):
        return [self.attn, self.toy]

    def cache_needs(self):
        return self.attn.cache_needs() + self.toy.cache_needs()

    def forward(self, x, ctx, caches):
        pages, state = caches
        return self.attn.forward(x, ctx, pages) + self.toy.forward(x, ctx, state)


def toy_spec(config):
    d, D = config.d_model, config.head_dim
    norm = lambda p: PartSpec("rmsnorm", p, {"dim": d, "eps": config.rms_norm_eps})
    ffn = lambda p: PartSpec("swiglu", p, {"d_model": d, "hidden": config.hidden_size, "bias": False})
    rope = PartSpec("rope", "", {"dim": D, "base": config.rope_theta, "style": "interleaved"})

    def attn(p, **kw):
        return PartSpec("attention", p, {"d_model": d, "num_heads": config.num_heads, "num_kv_heads": config.num_kv_heads,
                                         "head_dim": D, "position": rope, **kw})
    decay = config.extra.get("decay_kind", "toy_decay")
    mixers = [attn("layers.0.attn"), PartSpec(decay, "layers.1.toy", {"dim": d, "decay": 0.5}),
              attn("layers.2.attn", window=config.extra["window"], page_size=16), attn("layers.3.attn", shares_kv=True),
              PartSpec("toy_attention_plus_decay", "layers.4", {"attention": attn("layers.4.attn"),
                                                                "decay": PartSpec(decay, "layers.4.toy", {"dim": d, "decay": 0.5})})]
    layers = [LayerSpec(PartSpec("pre_norm", f"layers.{i}", {"mixer_norm": norm(f"layers.{i}.n1"), "mixer": m,
                                                              "ffn_norm": norm(f"layers.{i}.n2"), "ffn": ffn(f"layers.{i}.mlp")}))
              for i, m in enumerate(mixers)]
    # layer 0 runs twice (each run with a cache of its own); layer 3 reads the cache of the first run of layer 0
    # and layer 4's mixer keeps pages and a state
    order = (RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(0), RunEntry(3, cache_from=0), RunEntry(4))
    return ModelSpec(d_model=d, vocab_size=config.vocab_size, max_seq_len=config.max_seq_len,
                     embedding=PartSpec("token", "emb", {"vocab_size": config.vocab_size, "dim": d}),
                     layers=tuple(layers), run_order=order, final_norm=norm("final_norm"),
                     head=PartSpec("linear", "lm_head", {"dim": d, "vocab_size": config.vocab_size}))


def toy_plain_forward(cfg, w, tokens):
    """The toy architecture written out plainly, whole sequence, no cache."""
    w = {k: v.float() for k, v in w.items()}
    S, d, Hq, Hkv = len(tokens), cfg["d_model"], cfg["num_heads"], cfg["num_kv_heads"]
    D, eps = d // Hq, cfg["rms_norm_eps"]
    x = w["emb.weight"][torch.tensor(tokens)]
    cos, sin = pm.plain_rope_tables(D, torch.arange(S), cfg["rope_theta"])
    kept = {}

    def attn(h, p, window=None, kv=None, keep=None):
        q = pm.plain_rope((h @ w[f"{p}.q_proj.weight"].T).view(S, Hq, D), cos, sin)
        if kv is None:
            k = pm.plain_rope((h @ w[f"{p}.k_proj.weight"].T).view(S, Hkv, D), cos, sin)
            v = (h @ w[f"{p}.v_proj.weight"].T).view(S, Hkv, D)
        else:
            k, v = kv
        if keep:
            kept[keep] = (k, v)
        return pm.plain_attention(q, k, v, 1 / math.sqrt(D), window).reshape(S, d) @ w[f"{p}.out.weight"].T

    def toy(h, p):
        u, s, ys = h @ w[f"{p}.mix.weight"].T, torch.zeros(d), []
        for t in range(S):
            s = 0.5 * s + u[t]
            ys.append(s)
        return torch.stack(ys)

    def block(x, i, mixer):
        x = x + mixer(pm.plain_rmsnorm(x, w[f"layers.{i}.n1.weight"], eps))
        return x + pm.plain_swiglu(pm.plain_rmsnorm(x, w[f"layers.{i}.n2.weight"], eps), w, f"layers.{i}.mlp")

    x = block(x, 0, lambda h: attn(h, "layers.0.attn", keep="first"))
    x = block(x, 1, lambda h: toy(h, "layers.1.toy"))
    x = block(x, 2, lambda h: attn(h, "layers.2.attn", window=cfg["window"]))
    x = block(x, 0, lambda h: attn(h, "layers.0.attn"))
    x = block(x, 3, lambda h: attn(h, "layers.3.attn", kv=kept["first"]))
    x = block(x, 4, lambda h: attn(h, "layers.4.attn") + toy(h, "layers.4.toy"))
    return pm.plain_rmsnorm(x, w["final_norm.weight"], eps) @ w["lm_head.weight"].T


TOY_CFG = dict(architecture="toy_mix", vocab_size=300, d_model=80, num_layers=5, num_heads=5, num_kv_heads=1,
               hidden_size=112, max_seq_len=256, rope_theta=3000.0, rms_norm_eps=1e-5, window=21)


@pytest.fixture
def toy_registered():
    register_part("mixer", "toy_decay")(ToyDecayMixer)
    register_part("mixer", "toy_host_decay")(ToyHostDecayMixer)
    register_part("mixer", "toy_attention_plus_decay")(ToyAttentionPlusDecay)
    register_model("toy_mix")(toy_spec)
    yield
    unregister_model("toy_mix")
    unregister_part("mixer", "toy_attention_plus_decay")
    unregister_part("mixer", "toy_host_decay")
    unregister_part("mixer", "toy_decay")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "decode", "portions", "mixed"])
def test_toy_architecture_is_built_and_stepped(toy_registered, dtype, mode):
    cfg = dict(TOY_CFG)
    mc = ModelConfig.from_dict(cfg)
    assert mc.extra == {"window": 21}
    w = random_tensors(mc, 3, perturb_norms=True)
    assert "layers.1.toy.mix.weight" in w and "layers.3.attn.k_proj.weight" not in w and "layers.4.toy.mix.weight" in w
    g = torch.Generator().manual_seed(8)
    reqs = {f"r{i}": torch.randint(0, 300, (n,), generator=g).tolist() for i, n in enumerate((70, 150, 33, 256, 90))}
    steps = {"whole": tu.whole, "decode": tu.prefill_then_decode, "portions": tu.portions, "mixed": tu.mixed}[mode](reqs)
    page = 8
    ec = EngineConfig(dtype=dtype, device=DEV, use_cuda_graphs=False,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=tu.max_live_tokens(steps) // page + 1),
                      sched=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64))
    eng = Engine(mc, w, ec)
    # four runs own pages: three full-attention runs share a group, the windowed run has its own - with pages of its
    # own size and as many of them as hold the same tokens; two runs keep a state
    assert [len(g_.entries) for g_ in eng.manager.groups] == [3, 1] and sorted(eng.manager.entry_state) == [(1, 0), (5, 1)]
    assert [g_.page_size for g_ in eng.manager.groups] == [8, 16]
    assert eng.manager.groups[1].num_pages == -(-(eng.manager.groups[0].num_pages - 1) * 8 // 16) + 1
    exp = {rid: toy_plain_forward(cfg, w, toks) for rid, toks in reqs.items()}
    got = tu.run_steps(eng, steps)
    bad = tu.first_wrong(got, exp, TOL[dtype])
    assert bad is None, f"first wrong place {bad}"


def toy_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(toy_plain_forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("pipelined", [False, True])
def test_toy_architecture_generates_from_captured_graphs(toy_registered, pipelined):
    """The toy architecture - a windowed cache group, a state of fixed size, a mixer with two needs - through
    Engine.generate with captured decode steps (and the next step launched ahead of the host): the step that
    captures a graph must advance the per-request state once, and a windowed group must not stop the pipeline.
    Greedy tokens equal the architecture written out plainly."""
    cfg = dict(TOY_CFG)
    mc = ModelConfig.from_dict(cfg)
    w = random_tensors(mc, 3, std=0.3, perturb_norms=True)           # weights large enough for decided argmaxes
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 300, (n,), generator=g).tolist() for n in (30, 7, 55)]
    from tiny_transformer_inference_engine_b200 import SamplingParams
    ec = EngineConfig(dtype="float32", device=DEV, use_cuda_graphs=True, pipelined_decode=pipelined,
                      cache=CacheConfig(block_size=8, num_gpu_blocks=64),
                      sched=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=32, cudagraph_batch_sizes=[1, 2, 4]))
    eng = Engine(mc, w, ec)
    assert eng.model.capturable == "decode" and not eng.stepper.capture_repeated
    new = [40, 26, 33]                                                # requests end at different steps: the batch bucket changes
    out = eng.generate(prompts, [SamplingParams(max_new_tokens=n, greedy=True) for n in new])
    assert eng.stepper.counters["graph_replays"] > 20 and len(eng.stepper._graphs) >= 2
    for p, o, n in zip(prompts, out, new):
        assert o == toy_greedy(cfg, w, p, n)
    eng.manager.check()
    assert all(g_.allocator.num_free == g_.allocator.num_usable for g_ in eng.manager.groups)


def test_a_part_that_cannot_be_captured_keeps_the_model_off_graphs(toy_registered):
    cfg = dict(TOY_CFG, decay_kind="toy_host_decay")
    mc = ModelConfig.from_dict(cfg)
    w = random_tensors(mc, 3, std=0.3, perturb_norms=True)
    from tiny_transformer_inference_engine_b200 import SamplingParams
    ec = EngineConfig(dtype="float32", device=DEV, use_cuda_graphs=True, cache=CacheConfig(block_size=8, num_gpu_blocks=40),
                      sched=SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=32, cudagraph_batch_sizes=[1, 2]))
    eng = Engine(mc, w, ec)
    assert not eng.model.capturable and eng.stepper.graph_batch_sizes == []
    prompt = list(range(3, 20))
    assert eng.generate([prompt], SamplingParams(max_new_tokens=12, greedy=True))[0] == toy_greedy(cfg, w, prompt, 12)
    assert eng.stepper.counters["graph_replays"] == 0


# ------------------------------------------------------------------------------------------ more toy parts
class ToyRoutedFFN(FeedForward):
    """A feed-forward with routing: a router picks one of E small two-layer experts per token (router logits and
    their softmax in 32-bit); the output is the chosen expert's, scaled by its probability."""

    def __init__(self, prefix, d_model, hidden, experts):
        super().__init__(prefix)
        self.d, self.h, self.E = d_model, hidden, experts

    def param_specs(self):
        specs = {"router.weight": ParamSpec((self.E, self.d))}
        for e in range(self.E):
            specs[f"experts.{e}.up.weight"] = ParamSpec((self.h, self.d))
            specs[f"experts.{e}.down.weight"] = ParamSpec((self.d, self.h))
        return specs

    def load(self, params):
        self.router = params["router.weight"]
        self.up = [params[f"experts.{e}.up.weight"] for e in range(self.E)]
        self.down = [params[f"experts.{e}.down.weight"] for e in range(self.E)]

    def forward(self, x, ctx):
        probs = torch.softmax(x.float() @ self.router.float().T, -1)
        gate, choice = probs.max(-1)
        y = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e in range(self.E):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(self.ops.linear(x[rows].contiguous(), self.up[e], None))
                y[rows] = self.ops.linear(h, self.down[e], None).float() * gate[rows, None]
        return y.to(x.dtype)


class ToyOffsetPosition(PositionEncoding):
    """A position encoding that is no rotation: queries and keys get a fixed sinusoid of their position added
    (the general ``apply`` path of the attention part: no fused rotate-and-store)."""

    def __init__(self, prefix, dim, period):
        super().__init__(prefix)
        self.dim, self.period = dim, period

    def offsets(self, positions):
        i = torch.arange(self.dim, device=positions.device, dtype=torch.float32)
        return 0.3 * torch.sin(positions.float()[:, None] / self.period + i[None, :])

    def apply(self, q, k, positions):
        off = self.offsets(positions)[:, None, :]
        q.copy_((q.float() + off).to(q.dtype))
        if k is not None:
            k.copy_((k.float() + off).to(k.dtype))


def routed_spec(config):
    d, D = config.d_model, config.head_dim
    norm = lambda p: PartSpec("rmsnorm", p, {"dim": d, "eps": config.rms_norm_eps})
    pos = PartSpec("toy_offset", "", {"dim": D, "period": config.extra["period"]})
    layers = []
    for i in range(config.num_layers):
        attn = PartSpec("attention", f"layers.{i}.attn", {"d_model": d, "num_heads": config.num_heads,
                                                           "num_kv_heads": config.num_kv_heads, "head_dim": D, "position": pos})
        ffn = (PartSpec("toy_routed", f"layers.{i}.moe", {"d_model": d, "hidden": config.hidden_size, "experts": config.extra["experts"]})
               if i % 2 == 0 else PartSpec("swiglu", f"layers.{i}.mlp", {"d_model": d, "hidden": config.hidden_size, "bias": False}))
        layers.append(LayerSpec(PartSpec("pre_norm", f"layers.{i}", {"mixer_norm": norm(f"layers.{i}.n1"), "mixer": attn,
                                                                      "ffn_norm": norm(f"layers.{i}.n2"), "ffn": ffn})))
    return ModelSpec(d_model=d, vocab_size=config.vocab_size, max_seq_len=config.max_seq_len,
                     embedding=PartSpec("token", "emb", {"vocab_size": config.vocab_size, "dim": d}),
                     layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(config.num_layers)),
                     final_norm=norm("final_norm"), head=PartSpec("linear", "lm_head", {"dim": d, "vocab_size": config.vocab_size}))


def routed_plain_forward(cfg, w, tokens):
    """The routed toy architecture written out plainly, whole sequence, no cache."""
    w = {k: v.float() for k, v in w.items()}
    S, d, Hq, Hkv, E = len(tokens), cfg["d_model"], cfg["num_heads"], cfg["num_kv_heads"], cfg["experts"]
    D, eps = d // Hq, cfg["rms_norm_eps"]
    x = w["emb.weight"][torch.tensor(tokens)]
    i = torch.arange(D, dtype=torch.float32)
    off = (0.3 * torch.sin(torch.arange(S).float()[:, None] / cfg["period"] + i[None, :]))[:, None, :]
    for li in range(cfg["num_layers"]):
        h = pm.plain_rmsnorm(x, w[f"layers.{li}.n1.weight"], eps)
        p = f"layers.{li}.attn"
        q = (h @ w[f"{p}.q_proj.weight"].T).view(S, Hq, D) + off
        k = (h @ w[f"{p}.k_proj.weight"].T).view(S, Hkv, D) + off
        v = (h @ w[f"{p}.v_proj.weight"].T).view(S, Hkv, D)
        x = x + pm.plain_attention(q, k, v, 1 / math.sqrt(D), None).reshape(S, d) @ w[f"{p}.out.weight"].T
        h = pm.plain_rmsnorm(x, w[f"layers.{li}.n2.weight"], eps)
        if li % 2 == 0:
            p = f"layers.{li}.moe"
            probs = torch.softmax(h @ w[f"{p}.router.weight"].T, -1)
            gate, choice = probs.max(-1)
            y = torch.stack([torch.relu(h[t] @ w[f"{p}.experts.{int(choice[t])}.up.weight"].T)
                             @ w[f"{p}.experts.{int(choice[t])}.down.weight"].T * gate[t] for t in range(S)])
            x = x + y
        else:
            x = x + pm.plain_swiglu(h, w, f"layers.{li}.mlp")
    return pm.plain_rmsnorm(x, w["final_norm.weight"], eps) @ w["lm_head.weight"].T


@pytest.fixture
def routed_registered():
    register_part("ffn", "toy_routed")(ToyRoutedFFN)
    register_part("position", "toy_offset")(ToyOffsetPosition)
    register_model("toy_routed_model")(routed_spec)
    yield
    unregister_model("toy_routed_model")
    unregister_part("position", "toy_offset")
    unregister_part("ffn", "toy_routed")


@pytest.mark.parametrize("mode", ["whole", "decode", "portions", "mixed"])
def test_routed_ffn_and_other_position_encoding(routed_registered, mode):
    """A feed-forward with routing in every other layer and a position encoding that is no rotation, both defined
    here and registered without a change to the package: built from config.json keys, random weights by their
    tensor names, and stepped in every way of cutting against the architecture written out plainly.  (float32:
    a router's choice between near-equal experts must not depend on rounding.)"""
    cfg = dict(architecture="toy_routed_model", vocab_size=211, d_model=96, num_layers=3, num_heads=6, num_kv_heads=2,
               hidden_size=40, max_seq_len=200, rms_norm_eps=1e-5, rope_theta=1.0, experts=3, period=7.5)
    mc = ModelConfig.from_dict(cfg)
    assert mc.extra == {"experts": 3, "period": 7.5}
    w = random_tensors(mc, 4, std=0.1, perturb_norms=True)
    assert "layers.0.moe.experts.2.down.weight" in w and "layers.1.mlp.gate_proj.weight" in w and "layers.1.moe.router.weight" not in w
    g = torch.Generator().manual_seed(3)
    reqs = {f"r{i}": torch.randint(0, 211, (n,), generator=g).tolist() for i, n in enumerate((60, 133, 17, 200, 75))}
    steps = {"whole": tu.whole, "decode": tu.prefill_then_decode, "portions": tu.portions, "mixed": tu.mixed}[mode](reqs)
    page = 16
    ec = EngineConfig(dtype="float32", device=DEV, use_cuda_graphs=False,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=tu.max_live_tokens(steps) // page + 1),
                      sched=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64))
    eng = Engine(mc, w, ec)
    exp = {rid: routed_plain_forward(cfg, w, toks) for rid, toks in reqs.items()}
    got = tu.run_steps(eng, steps)
    bad = tu.first_wrong(got, exp, TOL["float32"])
    assert bad is None, f"first wrong place {bad}"
