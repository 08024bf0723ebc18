"""Each part alone against the plain functions, and the generality of the arrangement:
a toy mixer with state of its own, a layer that runs twice, a layer that reads another
layer's cache (needs a GPU)."""
import math
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

from helpers import assert_logits_close, random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTS = [torch.float32, torch.bfloat16]
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


def tol(dt):
    return dict(atol=2e-5, rtol=1e-4) if dt == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def close(got, ref, dt):
    """32-bit: element-wise; bfloat16: within 2 % of the largest reference value."""
    if dt == torch.float32:
        torch.testing.assert_close(got, ref, atol=2e-5, rtol=1e-4)
    else:
        bound = 2e-2 * float(ref.abs().max())
        worst = float((got - ref).abs().max())
        assert worst <= bound, f"largest difference {worst:.4g} exceeds {bound:.4g}"


def rnd(*shape, dt=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dt).to(DEV)


def context(dt, requests, starts, vocab=1 << 20, parts=()):
    """A StepContext for parts tested outside a model (``parts``: those whose host tables the step must carry)."""
    from rocmforge_b200.engine import Options, StepBatch, StepContext, StepRequest
    from rocmforge_b200.engine.batch import DeviceDescriptor
    pool = {}

    def scratch(name, n, dtype):
        return pool.setdefault((name, n, dtype), torch.zeros((max(n, 1),), dtype=dtype, device=DEV))
    fake_model = SimpleNamespace(options=Options(), compute_dtype=dt, device=torch.device(DEV), scratch=scratch)
    tables = {name: (lambda b, part=part, name=name: part.step_table(name, b))
              for part in parts for name in part.step_table_names()}
    batch = StepBatch([StepRequest(*r) for r in requests], starts, vocab, tables=tables)
    desc = DeviceDescriptor(DEV)
    desc.upload(batch.pack())
    ctx = StepContext(fake_model, desc.views(batch.T, batch.B, batch.R, batch.extras), T=batch.T, B=batch.B, R=batch.R,
                      is_decode=batch.is_decode, max_new=batch.max_new, max_end=batch.max_end, host=batch)
    ctx._keep = desc
    return ctx


@pytest.mark.parametrize("dt", DTS)
def test_rmsnorm_part_consumes_the_pending_update(dt):
    from rocmforge_b200.engine import ResidualStream
    from rocmforge_b200.parts import NORMS
    norm = NORMS.build("rmsnorm", size=200, eps=1e-4)
    assert list(norm.param_specs()) == ["weight"] and norm.param_specs()["weight"].kind == "vector"
    w = rnd(200, seed=1) + 1
    norm.bind({"weight": w}, dt)
    h, upd = rnd(6, 200, seed=2), rnd(6, 200, dt=dt, seed=3)
    stream = ResidualStream(h.clone())
    stream.add_pending(upd)
    y = norm.forward(None, stream)
    total = h.double() + upd.double()
    assert stream.pending is None
    torch.testing.assert_close(stream.h.double(), total, atol=1e-5, rtol=1e-6)
    torch.testing.assert_close(y.double(), P.rms_norm(total, w.double(), 1e-4), **tol(dt))


@pytest.mark.parametrize("dt", DTS)
def test_gated_mlp_part(dt):
    from rocmforge_b200.engine import ResidualStream
    from rocmforge_b200.parts import FEED_FORWARDS
    H, I, T = 72, 200, 11
    ffn = FEED_FORWARDS.build("gated_mlp", hidden=H, intermediate=I)
    p = {"gate_proj.weight": rnd(I, H, dt=dt, seed=1, scale=0.1), "up_proj.weight": rnd(I, H, dt=dt, seed=2, scale=0.1),
         "down_proj.weight": rnd(H, I, dt=dt, seed=3, scale=0.1)}
    assert {k: v.shape for k, v in ffn.param_specs().items()} == {k: tuple(v.shape) for k, v in p.items()}
    ffn.bind(p, dt)
    ctx = context(dt, [(0, [1] * T, [])], [0])
    y = rnd(T, H, dt=dt, seed=4)
    stream = ResidualStream(torch.zeros(T, H, device=DEV))
    ffn.forward(ctx, y, stream)
    ref = P.swiglu_mlp(y.double(), *(p[k].double() for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    torch.testing.assert_close(stream.flush().double(), ref, **tol(dt))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("window", [None, 40])
def test_attention_part_over_its_cache(dt, window):
    """A prompt, then a chunk, then single tokens, for two sequences of unequal length."""
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.engine import ResidualStream
    from rocmforge_b200.parts import MIXERS, POSITIONS
    H, nh, nkv, hd = 56, 6, 2, 16
    mixer = MIXERS.build("gqa_attention", hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=True,
                         window=window, position=POSITIONS.build("rope_neox", head_dim=hd, theta=1234.0))
    p = {}
    for i, (name, spec) in enumerate(mixer.param_specs().items()):
        p[name] = rnd(*spec.shape, dt=dt if spec.kind == "matrix" else torch.float32, seed=i, scale=0.2)
    mixer.bind(p, dt)
    cache = SequenceCache({0: mixer.cache_request()}, max_tokens=512, dtype=dt, device=DEV)
    lens = [150, 90]
    ys = [rnd(n, H, dt=dt, seed=10 + i) for i, n in enumerate(lens)]
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, hidden_size=H, rope_theta=1234.0,
               use_sliding_window=window is not None, sliding_window=window, max_window_layers=0)
    refs = [P.attention_block(y.double().cpu(), torch.arange(n), {"x." + k: v.double().cpu() for k, v in p.items()},
                              "x.", cfg, 0) for y, n in zip(ys, lens)]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    done = [0, 0]
    for chunk in ([100, 17], [30, 1], [1, 1], [19, 71]):
        reqs = [(s, [0] * n, []) for s, n in zip(slots, chunk)]
        cache.prepare(slots, chunk)
        ctx = context(dt, reqs, done, parts=[mixer])
        y = torch.cat([ys[i][done[i]:done[i] + n] for i, n in enumerate(chunk)])
        stream = ResidualStream(torch.zeros(sum(chunk), H, device=DEV))
        mixer.forward(ctx, y, cache.view(0), stream)
        cache.commit(slots, chunk)
        out = stream.flush().double().cpu()
        off = 0
        for i, n in enumerate(chunk):
            close(out[off:off + n], refs[i][done[i]:done[i] + n], dt)
            off += n
            done[i] += n
    assert done == lens


@pytest.mark.parametrize("dt", DTS)
def test_prenorm_block_alone(dt):
    """The arrangement itself: x += mixer(norm1(x)); x += ffn(norm2(x)), against the plain layer."""
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.engine import ResidualStream
    from rocmforge_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
    H, nh, nkv, hd, I, T = 48, 3, 3, 16, 72, 37
    block = BLOCKS.build(
        "prenorm", norm1=NORMS.build("rmsnorm", size=H, eps=1e-5),
        mixer=MIXERS.build("gqa_attention", hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=True,
                           position=POSITIONS.build("rope_neox", head_dim=hd, theta=777.0)),
        norm2=NORMS.build("rmsnorm", size=H, eps=1e-5), ffn=FEED_FORWARDS.build("gated_mlp", hidden=H, intermediate=I),
        names={"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.", "ffn": "mlp."})
    tensors = {}
    for prefix, part in block.sub_parts().items():
        local = {}
        for i, (name, spec) in enumerate(part.param_specs().items()):
            t = rnd(*spec.shape, dt=dt if spec.kind == "matrix" else torch.float32, seed=len(tensors) + i, scale=0.15)
            if spec.init == "ones":
                t = t + 1
            local[name] = t
            tensors["model.layers.0." + prefix + name] = t.double().cpu()
        part.bind(local, dt)
    cache = SequenceCache({0: block.mixer.cache_request()}, max_tokens=128, dtype=dt, device=DEV)
    slot = cache.alloc_slot()
    cache.prepare([slot], [T])
    ctx = context(dt, [(slot, [0] * T, [])], [0])
    x = rnd(T, H, seed=99)
    stream = ResidualStream(x.clone())
    block.forward(ctx, stream, cache.view(0))
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, hidden_size=H, rope_theta=777.0,
               rms_norm_eps=1e-5, use_sliding_window=False)
    ref = P.decoder_layer(x.double().cpu(), torch.arange(T), tensors, cfg, 0)
    close(stream.flush().double().cpu(), ref, dt)


@pytest.mark.parametrize("dt", DTS)
def test_embedding_and_head_parts(dt):
    from rocmforge_b200.parts import OutputHead, TokenEmbedding
    emb, head = TokenEmbedding(333, 40), OutputHead(333, 40, tied_to="model.embed_tokens.weight")
    w = rnd(333, 40, dt=dt, seed=1)
    emb.bind({"weight": w}, dt)
    head.bind({"weight": w}, dt)
    assert head.param_specs()["weight"].tied_to == "model.embed_tokens.weight"
    ids = torch.tensor([5, 332, 0], dtype=torch.int32, device=DEV)
    x = emb.forward(None, ids)
    assert x.dtype == torch.float32 and torch.equal(x, w[ids.long()].float())
    ctx = context(dt, [(0, [1, 2, 3], [])], [0])
    y = rnd(3, 40, dt=dt, seed=2)
    logits = head.forward(ctx, y)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.double(), y.double() @ w.double().t(), **tol(dt))


# --------------------------------------------------------------------------- generality of the arrangement

def scheduled_plain_logits(cfg, tensors, tokens, schedule):
    """Plain forward for a schedule of (layer, kv_from): a layer may run twice; an execution with
    kv_from attends with its own queries over the keys and values that execution kv_from made."""
    p = {k: v.double() for k, v in tensors.items()}
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], P.head_dim_of(cfg)
    T = len(tokens)
    pos = torch.arange(T)
    x = P.embedding(p["model.embed_tokens.weight"], torch.tensor(tokens))
    kept = {}
    for e, (layer, kv_from) in enumerate(schedule):
        pre = f"model.layers.{layer}."
        a = pre + "self_attn."
        y = P.rms_norm(x, p[pre + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q = P.rope_neox(P.linear(y, p[a + "q_proj.weight"], p[a + "q_proj.bias"]).view(T, nh, hd), pos, cfg["rope_theta"])
        if kv_from is None:
            k = P.rope_neox(P.linear(y, p[a + "k_proj.weight"], p[a + "k_proj.bias"]).view(T, nkv, hd), pos, cfg["rope_theta"])
            v = P.linear(y, p[a + "v_proj.weight"], p[a + "v_proj.bias"]).view(T, nkv, hd)
            kept[e] = (k, v)
        else:
            k, v = kept[kv_from]
        o = P.causal_attention(q, k, v)
        x = x + P.linear(o.reshape(T, nh * hd), p[a + "o_proj.weight"])
        y = P.rms_norm(x, p[pre + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + P.swiglu_mlp(y, p[pre + "mlp.gate_proj.weight"], p[pre + "mlp.up_proj.weight"], p[pre + "mlp.down_proj.weight"])
    x = P.rms_norm(x, p["model.norm.weight"], cfg["rms_norm_eps"])
    return P.linear(x, p["model.embed_tokens.weight"])


@pytest.mark.parametrize("dt", DTS)
def test_schedule_runs_a_layer_twice_and_shares_a_cache(folders, dt):
    import rocmforge_b200 as rf
    from rocmforge_b200.config import load_config
    from rocmforge_b200.weights import load_folder
    folder = folders("A", NAME[dt])
    arch, cfg = load_config(folder)
    spec = arch.build(cfg)
    schedule = [(0, None), (1, None), (1, None), (0, 1)]        # layer 1 twice; the last run reads entry 1's cache
    spec.schedule = [rf.ScheduleEntry(layer=l, kv_from=k) for l, k in schedule]
    assert sorted(spec.cache_requests()) == [0, 1, 2]           # the sharing execution owns no cache
    m = rf.Model(spec, load_folder(folder, spec.param_specs(), dt, DEV), dt, DEV)
    cache = m.new_cache(max_tokens=256)
    assert cache.groups[0].storage.shape[0] == 3
    plain_cfg, tensors = P.read_folder(folder)
    toks = random_tokens(256, 80, 3)
    ref = scheduled_plain_logits(plain_cfg, tensors, toks, schedule)
    s = cache.alloc_slot()
    got = [m.step(cache, [rf.StepRequest(s, toks[:70], range(70))]).cpu()]
    for t in toks[70:]:
        got.append(m.step(cache, [rf.StepRequest(s, [t], [0])]).cpu())
    assert_logits_close(torch.cat(got), ref, NAME[dt], "scheduled model")
    with pytest.raises(ValueError):
        spec.schedule = [rf.ScheduleEntry(0, kv_from=0)]
        spec.cache_requests()


def test_a_toy_mixer_with_state_registers_builds_and_steps():
    """A mixer defined here, with fixed-size per-sequence state (a decaying sum), becomes a model
    through the registries alone: no file of the framework changes."""
    import rocmforge_b200 as rf
    from rocmforge_b200.cache import StateRequest
    from rocmforge_b200.config import register_architecture
    from rocmforge_b200.engine import ModelSpec, ScheduleEntry
    from rocmforge_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Mixer, OutputHead, TokenEmbedding
    from rocmforge_b200.weights import ParamSpec

    @MIXERS.register("toy_decaying_sum")
    class DecayingSum(Mixer):
        """s_t = decay * s_{t-1} + W_in y_t;  update = W_out s_t."""

        def __init__(self, hidden, width, decay):
            self.hidden, self.width, self.decay = hidden, width, decay

        def param_specs(self):
            return {"in_proj.weight": ParamSpec((self.width, self.hidden), std=0.3),
                    "out_proj.weight": ParamSpec((self.hidden, self.width), std=0.3)}

        def bind(self, params, compute_dtype):
            self.w_in, self.w_out = params["in_proj.weight"], params["out_proj.weight"]

        def cache_request(self):
            return StateRequest.of(s=((self.width,), torch.float32))

        def forward(self, ctx, y, state, stream):
            u = ctx.matmul(y, self.w_in, out_f32=True)                      # the framework's product
            if ctx.is_decode:
                # one token per sequence: the state rows of the step's slots, indexed on the device (the batch's host
                # arrays do not exist inside a replayed graph)
                rows = ctx.seq_slot.long()
                out = state["s"][rows] * self.decay + u
                state["s"].index_copy_(0, rows, out)
            else:
                out = torch.empty_like(u)
                b = ctx.host
                for i, slot in enumerate(b.slots):                          # the scan itself is plain torch
                    s = state["s"][slot]
                    for t in range(int(b.cu_q[i]), int(b.cu_q[i + 1])):
                        s.mul_(self.decay).add_(u[t])
                        out[t] = s
            ctx.matmul_residual(out.to(ctx.compute_dtype), self.w_out, None, stream)

    @dataclass
    class ToyConfig:
        architecture: str
        hidden_size: int
        width: int
        decay: float
        num_hidden_layers: int
        vocab_size: int

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["architectures"][0], raw["hidden_size"], raw["width"], raw["decay"],
                       raw["num_hidden_layers"], raw["vocab_size"])

    def build(cfg):
        blocks = [BLOCKS.build("prenorm", norm1=NORMS.build("rmsnorm", size=cfg.hidden_size, eps=1e-5),
                               mixer=MIXERS.build("toy_decaying_sum", hidden=cfg.hidden_size, width=cfg.width,
                                                  decay=cfg.decay),
                               norm2=NORMS.build("rmsnorm", size=cfg.hidden_size, eps=1e-5),
                               ffn=FEED_FORWARDS.build("gated_mlp", hidden=cfg.hidden_size, intermediate=40),
                               names={"norm1": "n1.", "mixer": "mix.", "norm2": "n2.", "ffn": "ff."})
                  for _ in range(cfg.num_hidden_layers)]
        return ModelSpec(config=cfg, embedding=TokenEmbedding(cfg.vocab_size, cfg.hidden_size), embedding_prefix="emb.",
                         blocks=blocks, block_prefixes=[f"l{i}." for i in range(cfg.num_hidden_layers)],
                         final_norm=NORMS.build("rmsnorm", size=cfg.hidden_size, eps=1e-5), final_norm_prefix="fn.",
                         head=OutputHead(cfg.vocab_size, cfg.hidden_size, tied_to="emb.weight"), head_prefix="head.",
                         schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
                         vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, max_position=4096)

    register_architecture("ToyStateLM", ToyConfig, build)
    cfg = ToyConfig.from_dict(dict(architectures=["ToyStateLM"], hidden_size=24, width=10, decay=0.8,
                                   num_hidden_layers=2, vocab_size=50))
    m = rf.Model.random(cfg, seed=4, dtype=torch.float32)
    cache = m.new_cache(max_tokens=256, max_slots=4)
    assert cache.groups == [] and sorted(cache.states) == [0, 1]
    toks = [random_tokens(50, n, n) for n in (30, 14)]
    # whole, alone
    whole = []
    for t in toks:
        s = cache.alloc_slot()
        whole.append(m.step(cache, [rf.StepRequest(s, t, range(len(t)))]).cpu())
        cache.free_slot(s)
    # the same two as a batch: prompts of unequal length, then one token each; state carries over,
    # and the reused slots start from zero state
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    got = m.step(cache, [rf.StepRequest(s, t[:5], range(5)) for s, t in zip(slots, toks)])
    torch.testing.assert_close(got[:5].cpu(), whole[0][:5], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(got[5:].cpu(), whole[1][:5], atol=1e-5, rtol=1e-4)
    for i in range(5, 7):
        got = m.step(cache, [rf.StepRequest(s, [t[i]], [0]) for s, t in zip(slots, toks)])
        torch.testing.assert_close(got[0].cpu(), whole[0][i], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(got[1].cpu(), whole[1][i], atol=1e-5, rtol=1e-4)
    # the same sequences go on through replayed graphs (logits, and sampled ids one step ahead of the host): the state
    # lives in device tensors indexed by the step's slots, so a captured step reads and writes the right rows
    from rocmforge_b200.engine.graph import DecodeRunner
    runner = DecodeRunner(m, cache)
    for i in range(7, 11):
        got = runner.logits(slots, [t[i] for t in toks]).cpu()
        torch.testing.assert_close(got[0], whole[0][i], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(got[1], whole[1][i], atol=1e-5, rtol=1e-4)
    greedy = rf.SamplingParams(temperature=0.0)
    for i in range(11, 14):
        ids = runner.step_ids(slots, [t[i] for t in toks], greedy, [0, 1], [i, i], more=False)
        assert ids == [int(whole[0][i].argmax()), int(whole[1][i].argmax())]
    assert runner.replays >= 7
    # and against the recurrence written out
    p = {n: t.double().cpu() for n, t in _params_of(m).items()}
    x = p["emb.weight"][torch.tensor(toks[1])]
    for l in range(2):
        y = P.rms_norm(x, p[f"l{l}.n1.weight"], 1e-5)
        u = y @ p[f"l{l}.mix.in_proj.weight"].t()
        s, outs = torch.zeros(10, dtype=torch.float64), []
        for t in range(len(u)):
            s = 0.8 * s + u[t]
            outs.append(s)
        x = x + torch.stack(outs) @ p[f"l{l}.mix.out_proj.weight"].t()
        y = P.rms_norm(x, p[f"l{l}.n2.weight"], 1e-5)
        x = x + P.swiglu_mlp(y, p[f"l{l}.ff.gate_proj.weight"], p[f"l{l}.ff.up_proj.weight"], p[f"l{l}.ff.down_proj.weight"])
    ref = P.rms_norm(x, p["fn.weight"], 1e-5) @ p["emb.weight"].t()
    torch.testing.assert_close(whole[1].double(), ref, atol=2e-5, rtol=1e-4)


def _params_of(model):
    """Tensors of a model by full name, gathered back from its bound parts (test helper)."""
    out = {}
    for prefix, part in model.spec.named_parts().items():
        for attr, name in (("weight", "weight"), ("w_in", "in_proj.weight"), ("w_out", "out_proj.weight")):
            if hasattr(part, attr) and isinstance(getattr(part, attr), torch.Tensor) and name in part.param_specs():
                out[prefix + name] = getattr(part, attr)
        if hasattr(part, "gate_up") and part.gate_up is not None:
            gu = part.gate_up.weight
            out[prefix + "gate_proj.weight"], out[prefix + "up_proj.weight"] = gu[0::2], gu[1::2]
            out[prefix + "down_proj.weight"] = part.down.weight
    return out


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_plug_in():
    """Two more kinds defined here and reached through the registries alone: a feed-forward that routes every
    token to one of several small experts (router logits in 32-bit), and a position encoding that stretches
    positions by a factor and turns only the first half of every head, neighbouring elements as pairs (it hands the
    rotation kernel its table of frequencies, its rotary size and its pairing); and a mixer without any encoding."""
    import rocmforge_b200 as rf
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.engine import ResidualStream
    from rocmforge_b200.parts import FEED_FORWARDS, MIXERS, POSITIONS, FeedForward, PositionEncoding
    from rocmforge_b200.weights import ParamSpec
    dt = torch.float32

    @FEED_FORWARDS.register("toy_top1_experts")
    class Top1Experts(FeedForward):
        def __init__(self, hidden, inner, n_experts):
            self.hidden, self.inner, self.n = hidden, inner, n_experts

        def param_specs(self):
            s = {"router.weight": ParamSpec((self.n, self.hidden), std=0.5)}
            for e in range(self.n):
                s[f"experts.{e}.up.weight"] = ParamSpec((self.inner, self.hidden), std=0.2)
                s[f"experts.{e}.down.weight"] = ParamSpec((self.hidden, self.inner), std=0.2)
            return s

        def bind(self, params, compute_dtype):
            self.p = params

        def forward(self, ctx, y, stream):
            logits = ctx.matmul(y, self.p["router.weight"], out_f32=True)           # 32-bit router logits
            choice = logits.argmax(dim=-1)
            gate = torch.softmax(logits, dim=-1).gather(1, choice[:, None])
            for e in range(self.n):                                                  # tokens of expert e, as one batch
                rows = torch.nonzero(choice == e)[:, 0]
                if rows.numel() == 0:
                    continue
                h = torch.relu(ctx.matmul(y[rows].contiguous(), self.p[f"experts.{e}.up.weight"]))
                upd = ctx.matmul(h, self.p[f"experts.{e}.down.weight"], out_f32=True) * gate[rows]
                stream.flush().index_add_(0, rows, upd)

    @POSITIONS.register("toy_stretched_rope")
    class StretchedRope(PositionEncoding):
        """Rotation by (position / factor) of the first ``rot`` elements of a head, pairs (2i, 2i+1)."""
        def __init__(self, head_dim, theta, factor, rot):
            self.rot = rot
            i = torch.arange(rot // 2, dtype=torch.float64)
            self.inv_freq_host = (1.0 / (theta ** (2.0 * i / rot)) / factor).to(torch.float32)
            self.inv_freq = None

        def prepare(self, device):
            self.inv_freq = self.inv_freq_host.to(device)

        def rotation(self):
            return dict(inv_freq=self.inv_freq, rot_dim=self.rot, interleaved=True)

    # ---- the routed feed-forward against the same thing written out
    H, I, E, T = 40, 24, 3, 50
    ffn = FEED_FORWARDS.build("toy_top1_experts", hidden=H, inner=I, n_experts=E)
    p = {n: rnd(*sp.shape, seed=i, scale=sp.std) for i, (n, sp) in enumerate(ffn.param_specs().items())}
    ffn.bind(p, dt)
    ctx = context(dt, [(0, [1] * T, [])], [0])
    y = rnd(T, H, seed=77)
    stream = ResidualStream(torch.zeros(T, H, device=DEV))
    ffn.forward(ctx, y, stream)
    yd = y.double().cpu()
    logits = yd @ p["router.weight"].double().cpu().t()
    ref = torch.zeros(T, H, dtype=torch.float64)
    for t in range(T):
        e = int(logits[t].argmax())
        g = torch.softmax(logits[t], dim=-1)[e]
        h = torch.relu(yd[t] @ p[f"experts.{e}.up.weight"].double().cpu().t())
        ref[t] = g * (h @ p[f"experts.{e}.down.weight"].double().cpu().t())
    torch.testing.assert_close(stream.flush().double().cpu(), ref, atol=2e-5, rtol=1e-4)
    assert len(set(int(logits[t].argmax()) for t in range(T))) == E, "every expert should get tokens in this test"

    # ---- the stretched rotation inside the framework's attention part
    nh, nkv, hd, factor, rot_dim = 4, 2, 16, 4.0, 8
    mixer = MIXERS.build("gqa_attention", hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=False,
                         position=POSITIONS.build("toy_stretched_rope", head_dim=hd, theta=100.0, factor=factor, rot=rot_dim))
    pm = {n: rnd(*sp.shape, seed=20 + i, scale=0.2) for i, (n, sp) in enumerate(mixer.param_specs().items())}
    mixer.bind(pm, dt)
    cache = SequenceCache({0: mixer.cache_request()}, max_tokens=128, dtype=dt, device=DEV)
    slot = cache.alloc_slot()
    cache.prepare([slot], [T])
    ctx = context(dt, [(slot, [0] * T, [])], [0])
    stream = ResidualStream(torch.zeros(T, H, device=DEV))
    mixer.forward(ctx, y, cache.view(0), stream)
    # plain: rotate by positions / factor (the plain rope takes integer positions, so stretch theta-free by hand)
    q = (yd @ pm["q_proj.weight"].double().cpu().t()).view(T, nh, hd)
    k = (yd @ pm["k_proj.weight"].double().cpu().t()).view(T, nkv, hd)
    v = (yd @ pm["v_proj.weight"].double().cpu().t()).view(T, nkv, hd)

    def rot(x):
        # pairs (2i, 2i+1) of the first rot_dim elements (maeddesg/ROCmForge src/cpu/ops.rs:86-96, neox=false)
        ang = (torch.arange(T, dtype=torch.float32)[:, None] * mixer.position.inv_freq_host[None, :]).double()
        c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = x.clone()
        x0, x1 = x[..., 0:rot_dim:2], x[..., 1:rot_dim:2]
        out[..., 0:rot_dim:2] = x0 * c - x1 * s_
        out[..., 1:rot_dim:2] = x0 * s_ + x1 * c
        return out
    o = P.causal_attention(rot(q), rot(k), v)
    ref = o.reshape(T, nh * hd) @ pm["o_proj.weight"].double().cpu().t()
    torch.testing.assert_close(stream.flush().double().cpu(), ref, atol=2e-5, rtol=1e-4)

    # ---- no position encoding at all: queries and keys go into the cache as they are
    bare = MIXERS.build("gqa_attention", hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=False, position=None)
    bare.bind(pm, dt)
    cache = SequenceCache({0: bare.cache_request()}, max_tokens=128, dtype=dt, device=DEV)
    slot = cache.alloc_slot()
    cache.prepare([slot], [T])
    ctx = context(dt, [(slot, [0] * T, [])], [0])
    stream = ResidualStream(torch.zeros(T, H, device=DEV))
    bare.forward(ctx, y, cache.view(0), stream)
    ref = P.causal_attention(q, k, v).reshape(T, nh * hd) @ pm["o_proj.weight"].double().cpu().t()
    torch.testing.assert_close(stream.flush().double().cpu(), ref, atol=2e-5, rtol=1e-4)


def test_a_model_whose_layers_differ_in_mixer_window_rotation_and_width():
    """One model, three kinds of layer: attention over a window of 24 keys with the whole head rotated; a mixer
    with per-sequence state and no cache of keys (defined here); attention over all keys with half of every head
    rotated; feed-forwards of three widths.  The cache gets a page group per need and a state tensor beside them;
    whole prompts, chunks, single tokens, an unequal batch and replayed graphs all give the logits of the same
    arithmetic written out."""
    import rocmforge_b200 as rf
    from rocmforge_b200.cache import StateRequest
    from rocmforge_b200.config import register_architecture
    from rocmforge_b200.engine import ModelSpec, ScheduleEntry
    from rocmforge_b200.engine.graph import DecodeRunner
    from rocmforge_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Mixer, OutputHead, TokenEmbedding
    from rocmforge_b200.weights import ParamSpec
    from test_kernels_gpu import plain_rotation
    H, nh, nkv, hd, V, eps, decay = 48, 4, 2, 16, 90, 1e-5, 0.7
    inters, windows, rots = (40, 24, 72), (24, None, None), (16, None, 8)

    @MIXERS.register("toy_leaky_state")
    class LeakyState(Mixer):
        """s_t = decay * s_{t-1} + y_t (the state is as wide as the model); update = W s_t."""
        def __init__(self, hidden):
            self.hidden = hidden

        def param_specs(self):
            return {"mix.weight": ParamSpec((self.hidden, self.hidden), std=0.2)}

        def bind(self, params, compute_dtype):
            self.w = params["mix.weight"]

        def cache_request(self):
            return StateRequest.of(s=((self.hidden,), torch.float32))

        def forward(self, ctx, y, state, stream):
            y32 = y.to(torch.float32)
            rows = ctx.seq_slot.long()
            if ctx.is_decode:
                out = state["s"][rows] * decay + y32
                state["s"].index_copy_(0, rows, out)
            else:
                out = torch.empty_like(y32)
                b = ctx.host
                for i, slot in enumerate(b.slots):
                    s = state["s"][slot]
                    for t in range(int(b.cu_q[i]), int(b.cu_q[i + 1])):
                        s.mul_(decay).add_(y32[t])
                        out[t] = s
            ctx.matmul_residual(out.to(ctx.compute_dtype), self.w, None, stream)

    @dataclass
    class MixedConfig:
        architecture: str

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["architectures"][0])

    def build(cfg):
        blocks = []
        for layer in range(3):
            if layer == 1:
                mixer = MIXERS.build("toy_leaky_state", hidden=H)
            else:
                mixer = MIXERS.build("gqa_attention", hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd, qkv_bias=layer == 0,
                                     window=windows[layer],
                                     position=POSITIONS.build("rope_neox", head_dim=hd, theta=500.0, rotary_dim=rots[layer]))
            blocks.append(BLOCKS.build("prenorm", norm1=NORMS.build("rmsnorm", size=H, eps=eps), mixer=mixer,
                                       norm2=NORMS.build("rmsnorm", size=H, eps=eps),
                                       ffn=FEED_FORWARDS.build("gated_mlp", hidden=H, intermediate=inters[layer]),
                                       names={"norm1": "n1.", "mixer": "mix.", "norm2": "n2.", "ffn": "ff."}))
        return ModelSpec(config=cfg, embedding=TokenEmbedding(V, H), embedding_prefix="emb.", blocks=blocks,
                         block_prefixes=[f"l{i}." for i in range(3)], final_norm=NORMS.build("rmsnorm", size=H, eps=eps),
                         final_norm_prefix="fn.", head=OutputHead(V, H, tied_to="emb.weight"), head_prefix="head.",
                         schedule=[ScheduleEntry(i) for i in range(3)], vocab_size=V, hidden_size=H, max_position=512)

    register_architecture("ToyMixedLM", MixedConfig, build)
    m = rf.Model.random(MixedConfig("ToyMixedLM"), seed=9, dtype=torch.float32)
    cache = m.new_cache(max_tokens=64 * 8, max_slots=4)
    assert sorted(g.window or 0 for g in cache.groups) == [0, 24] and sorted(cache.states) == [1]

    # ---- the same arithmetic written out
    dd = lambda t: t.double().cpu()
    def plain_logits(tokens):
        T = len(tokens)
        pos = torch.arange(T)
        x = dd(m.spec.embedding.weight)[torch.tensor(tokens)]
        for layer, blk in enumerate(m.spec.blocks):
            y = P.rms_norm(x, dd(blk.norm1.weight), eps)
            mx = blk.mixer
            if layer == 1:
                s, outs = torch.zeros(H, dtype=torch.float64), []
                for t in range(T):
                    s = decay * s + y[t]
                    outs.append(s)
                x = x + torch.stack(outs) @ dd(mx.w).t()
            else:
                qkv = y @ dd(mx.qkv.weight).t() + (dd(mx.qkv.bias) if mx.qkv.bias is not None else 0.0)
                q, k, v = qkv[:, :nh * hd].reshape(T, nh, hd), qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd), qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
                inv = mx.position.inv_freq_host
                q, k = plain_rotation(q, pos, inv, rots[layer], False), plain_rotation(k, pos, inv, rots[layer], False)
                o = P.causal_attention(q, k, v, window=windows[layer])
                x = x + o.reshape(T, nh * hd) @ dd(mx.o.weight).t()
            y = P.rms_norm(x, dd(blk.norm2.weight), eps)
            gu = dd(blk.ffn.gate_up.weight)
            x = x + P.swiglu_mlp(y, gu[0::2], gu[1::2], dd(blk.ffn.down.weight))
        return P.rms_norm(x, dd(m.spec.final_norm.weight), eps) @ dd(m.spec.embedding.weight).t()

    seqs = [random_tokens(V, n, 40 + n) for n in (100, 37, 70)]
    refs = [plain_logits(t) for t in seqs]
    # whole, alone
    for t, r in zip(seqs, refs):
        s = cache.alloc_slot()
        assert_logits_close(m.step(cache, [rf.StepRequest(s, t, range(len(t)))]).cpu(), r, "float32", "mixed model, whole")
        cache.free_slot(s)
    # an unequal batch: prompts in one step, a chunk each, single tokens, then replayed graphs; the shortest ends first
    slots = [cache.alloc_slot() for _ in seqs]
    at = [20, 5, 33]
    m.step(cache, [rf.StepRequest(s, t[:a], []) for s, t, a in zip(slots, seqs, at)])
    got = m.step(cache, [rf.StepRequest(s, t[a:a + 6], range(6)) for s, t, a in zip(slots, seqs, at)]).cpu()
    assert_logits_close(got, torch.cat([r[a:a + 6] for r, a in zip(refs, at)]), "float32", "mixed model, chunks")
    at = [a + 6 for a in at]
    runner = DecodeRunner(m, cache)
    live = [0, 1, 2]
    for step in range(60):
        for i in [i for i in live if at[i] >= len(seqs[i])]:
            cache.free_slot(slots[i]); live.remove(i)
        if not live:
            break
        toks = [seqs[i][at[i]] for i in live]
        if step < 8:
            got = m.step(cache, [rf.StepRequest(slots[i], [tk], [0]) for i, tk in zip(live, toks)]).cpu()
        else:
            got = runner.logits([slots[i] for i in live], toks).cpu()
        assert_logits_close(got, torch.stack([refs[i][at[i]] for i in live]), "float32", f"mixed model, step {step}")
        for i in live:
            at[i] += 1
    assert runner.replays > 20 and cache.live_slots == 1        # the longest sequence is still there
