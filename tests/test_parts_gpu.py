"""Each part alone against its plain counterpart; the schedule as data; a toy mixer with state
of its own, defined here, registered, built and stepped without touching the library."""
import dataclasses
import math

import numpy as np
import pytest
import torch

from helpers import REL, REL_CUT, load_plain, plain_logits, random_ids, rel_err
from plain import llama_plain as P
from tiny import TINY_A, TINY_B, make_model_dir

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype):
    from ithaca_b200.parts import Runtime
    return Runtime(dtype=dtype, device=DEV)


def one_sequence_context(n, start=0):
    from ithaca_b200.engine.context import ContextBuilder
    pages = -(-(start + n) // 64)
    table = np.arange(pages, dtype=np.int32)[None, :]
    return ContextBuilder(DEV).build([0], [list(range(n))], [start], [[]], [table])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from ithaca_b200.config import PartSpec
    from ithaca_b200.parts.norm import RMSNorm
    w = 1 + 0.1 * torch.randn(200)
    part = RMSNorm(PartSpec("rmsnorm", {"size": 200, "eps": 3e-6}, {"weight": "w"}), {"w": w.to(torch.bfloat16)}, runtime(dtype))
    x = torch.randn(5, 200) * 2
    got = part.forward(x.to(DEV)).double().cpu()
    ref = P.rmsnorm(x.double(), w.to(torch.bfloat16).double(), 3e-6)
    assert rel_err(got.numpy(), ref.numpy()) <= (2e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from ithaca_b200.config import PartSpec
    from ithaca_b200.parts.feed_forward import GatedMLP
    d, ff, T = 72, 172, 9
    t = {"g": torch.randn(ff, d) * 0.2, "u": torch.randn(ff, d) * 0.2, "d": torch.randn(d, ff) * 0.2}
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    part = GatedMLP(PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": ff, "activation": "silu"},
                             {"gate": "g", "up": "u", "down": "d"}), t, runtime(dtype))
    rt = runtime(dtype)
    x = torch.randn(T, d).to(rt.act_dtype)
    residual = torch.randn(T, d)
    res_dev = residual.to(DEV).clone()
    part.forward(x.to(DEV), None, res_dev)
    ref = residual.double() + P.gated_mlp(x.double(), t["g"], t["u"], t["d"])
    assert rel_err(res_dev.double().cpu().numpy(), ref.numpy()) <= (2e-6 if dtype == "float32" else 6e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_prompt_then_tokens(dtype, window):
    from ithaca_b200.cache import SequenceCache
    from ithaca_b200.config import PartSpec
    from ithaca_b200.engine.context import ContextBuilder
    from ithaca_b200.parts.attention import Attention
    from ithaca_b200.parts.position import RotaryPosition
    d, nh, nkv, hd, T = 80, 6, 3, 32, 75
    rt = runtime(dtype)
    names = {"q": "q", "k": "k", "v": "v", "o": "o"}
    t = {"q": torch.randn(nh * hd, d) * 0.2, "k": torch.randn(nkv * hd, d) * 0.2, "v": torch.randn(nkv * hd, d) * 0.2,
         "o": torch.randn(d, nh * hd) * 0.2}
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    pos = RotaryPosition(PartSpec("rotary", {"rotary_dim": hd, "theta": 1000.0, "pairing": "half", "scaling": None}), {}, rt)
    part = Attention(PartSpec("attention", {"hidden_size": d, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd,
                                            "window": window, "scale": None}, names), t, rt, position=pos)
    cache = SequenceCache({0: part.cache_requests()}, max_tokens=256, kv_dtype=rt.kv_dtype, device=DEV)
    slot = cache.alloc_slot()
    x = torch.randn(T, d).to(rt.act_dtype)
    # plain: the whole sequence at once
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "sliding_window": window,
           "use_sliding_window": window is not None}
    w = {f"p.{k}_proj.weight": v for k, v in t.items()}
    ref = P.attention_block(x.double(), w, "p", cfg, P.rope_inv_freq(hd, 1000.0, None), torch.arange(T))
    # part: 60 tokens in one step, then 15 one by one
    builder = ContextBuilder(DEV)
    out = torch.zeros(T, d, device=DEV)
    done = 0
    for n in [60] + [1] * 15:
        cache.reserve([slot], [n])
        ctx = builder.build([slot], [[0] * n], [done], [[]], [cache.table.table_rows(0, [slot], 2)])
        part.forward(x[done:done + n].to(DEV), ctx, cache.layer(0), out[done:done + n], True)
        cache.commit([slot], [n])
        done += n
    assert rt.status.item() == 0
    assert rel_err(out.double().cpu().numpy(), ref.numpy()) <= (3e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_arrangement(dtype, tmp_path):
    """One pre-norm block alone: x += attention(norm(x)); x += feed_forward(norm(x)), fed a residual stream
    of the test's own making, against the plain parts in the same order."""
    from ithaca_b200.cache import SequenceCache
    from ithaca_b200.config import config_from_model_dir
    from ithaca_b200.engine.context import ContextBuilder
    from ithaca_b200.parts import BLOCKS
    from ithaca_b200.weights import read_model_tensors
    d = make_model_dir(tmp_path, TINY_B, seed=6)
    pcfg, pt = load_plain(d)
    _, cfg = config_from_model_dir(d)
    spec = cfg.model_spec().layers[1]
    rt = runtime(dtype)
    block = BLOCKS.get(spec.kind)(spec, read_model_tensors(d), rt)
    cache = SequenceCache({0: block.cache_requests()}, max_tokens=128, kv_dtype=rt.kv_dtype, device=DEV)
    slot = cache.alloc_slot()
    T = 50
    x = torch.randn(T, 192) * 0.5
    res = x.to(DEV).clone()
    cache.reserve([slot], [T])
    ctx = ContextBuilder(DEV).build([slot], [[0] * T], [0], [[]], [cache.table.table_rows(0, [slot], 1)])
    block.forward(res, ctx, cache.layer(0), True)
    c = P.normalized_config(pcfg)
    p = "model.layers.1"
    xd = x.double()
    xn = P.rmsnorm(xd, pt[f"{p}.input_layernorm.weight"], c["rms_norm_eps"])
    xd = xd + P.attention_block(xn, pt, f"{p}.self_attn", c, P.rope_inv_freq(c["head_dim"], c["rope_theta"], c["rope_scaling"]),
                                torch.arange(T))
    xn = P.rmsnorm(xd, pt[f"{p}.post_attention_layernorm.weight"], c["rms_norm_eps"])
    xd = xd + P.gated_mlp(xn, pt[f"{p}.mlp.gate_proj.weight"], pt[f"{p}.mlp.up_proj.weight"], pt[f"{p}.mlp.down_proj.weight"])
    assert rt.status.item() == 0
    assert rel_err(res.double().cpu().numpy(), xd.numpy()) <= (3e-6 if dtype == "float32" else 5e-3)


def test_embedding_and_head_parts():
    from ithaca_b200.config import PartSpec
    from ithaca_b200.parts.embedding import Embedding, OutputHead
    rt = runtime("bfloat16")
    table = (torch.randn(301, 72) * 0.1).to(torch.bfloat16)
    emb = Embedding(PartSpec("embedding", {"vocab_size": 301, "hidden_size": 72, "scale": 1.0}, {"weight": "e"}), {"e": table}, rt)
    ids = torch.tensor([5, 300, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table.float()[[5, 300, 0]])
    head = OutputHead(PartSpec("lm_head", {"vocab_size": 301, "hidden_size": 72, "tied": True}, {"weight": "e"}), {"e": emb.table}, rt)
    assert head.linear.weight.data_ptr() == emb.table.data_ptr()                # a tied head shares the table on the device
    xn = (torch.randn(4, 72)).to(torch.bfloat16)
    got = head.forward(xn.to(DEV)).double().cpu()
    assert rel_err(got.numpy(), (xn.double() @ table.double().T).numpy()) <= 2e-5


def test_schedule_names_a_layer_twice_and_shares_a_cache(tmp_path):
    """The order of runs is data.  Layer 0 runs twice with caches of its own; a last run of layer 1
    reads the cache its first run filled.  The plain side spells the same order out by hand."""
    from ithaca_b200.cache import SequenceCache
    from ithaca_b200.config import ScheduleEntry, config_from_model_dir
    from ithaca_b200.engine.model import DecoderModel
    from ithaca_b200.engine.step import Stepper
    from ithaca_b200.weights import read_model_tensors
    d = make_model_dir(tmp_path, TINY_A, seed=4)
    pcfg, pt = load_plain(d)
    _, cfg = config_from_model_dir(d)
    spec = dataclasses.replace(cfg.model_spec(), schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                                                           ScheduleEntry(1, 1, writes_cache=False)))
    rt = runtime("float32")
    model = DecoderModel(spec, read_model_tensors(d), rt)
    cache = SequenceCache(model.cache_requests(), max_tokens=256, kv_dtype=rt.kv_dtype, device=DEV)
    assert len(cache.kv_groups) == 1 and cache.kv_groups[0].cache_entries == (0, 1, 2)
    st = Stepper(model, cache)
    ids = random_ids(40, 256, 9)
    s = cache.alloc_slot()
    got = torch.cat([st.step([s], [ids[:30]], "all")] + [st.step([s], [[t]], "last") for t in ids[30:]]).cpu().numpy()

    # plain: the same four runs; the fourth attends with its own queries over the keys/values of run 2
    c = P.normalized_config(pcfg)
    inv = P.rope_inv_freq(c["head_dim"], c["rope_theta"], None)
    pos = torch.arange(len(ids))
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    x = P.embed(ids, pt["model.embed_tokens.weight"])
    kept = {}
    for run, (layer, share) in enumerate([(0, None), (1, None), (0, None), (1, 1)]):
        p = f"model.layers.{layer}"
        xn = P.rmsnorm(x, pt[f"{p}.input_layernorm.weight"], c["rms_norm_eps"])
        q = P.rope((xn @ pt[f"{p}.self_attn.q_proj.weight"].double().T).view(-1, nh, hd), pos, inv)
        if share is None:
            k = P.rope((xn @ pt[f"{p}.self_attn.k_proj.weight"].double().T).view(-1, nkv, hd), pos, inv)
            v = (xn @ pt[f"{p}.self_attn.v_proj.weight"].double().T).view(-1, nkv, hd)
            kept[run] = (k, v)
        else:
            k, v = kept[share]
        att = P.attention(q, k, v).reshape(len(ids), nh * hd)
        x = x + att @ pt[f"{p}.self_attn.o_proj.weight"].double().T
        xn = P.rmsnorm(x, pt[f"{p}.post_attention_layernorm.weight"], c["rms_norm_eps"])
        x = x + P.gated_mlp(xn, pt[f"{p}.mlp.gate_proj.weight"], pt[f"{p}.mlp.up_proj.weight"], pt[f"{p}.mlp.down_proj.weight"])
    ref = (P.rmsnorm(x, pt["model.norm.weight"], c["rms_norm_eps"]) @ pt["lm_head.weight"].double().T).numpy()
    assert rel_err(got, ref) <= REL["float32"]


# ------------------------------------------------------------------------------------------ a toy mixer with state
class ToyDecayMixer:
    """state_t = decay * state_{t-1} + W_in x_t ; y_t = W_out state_t.  Its state is fixed-size,
    lives in the cache's state area, and must be carried across steps per slot."""

    @classmethod
    def manifest(cls, spec):
        from ithaca_b200.weights import TensorReq
        d, n = spec["hidden_size"], spec["state_size"]
        return {spec.weights["in"]: TensorReq((n, d)), spec.weights["out"]: TensorReq((d, n))}

    def __init__(self, spec, tensors, runtime):
        self.d, self.n, self.decay = spec["hidden_size"], spec["state_size"], spec["decay"]
        self.w_in = tensors[spec.weights["in"]].to(runtime.device).float()
        self.w_out = tensors[spec.weights["out"]].to(runtime.device).float()

    def cache_requests(self):
        from ithaca_b200.cache import StateRequest
        return [StateRequest("decay_state", (self.n,), "float32")]

    def forward(self, x, ctx, cache, residual, writes_cache=True):
        state = cache.state("decay_state")                     # [max_slots, n]
        u = x.float() @ self.w_in.T
        cu = [0] + list(np.cumsum(ctx.host_n_new))             # host copies: no device read-back
        for b, slot in enumerate(ctx.host_slots):              # tokens of a sequence in order, sequences by slot
            s = state[slot].clone()
            for t in range(cu[b], cu[b + 1]):
                s = self.decay * s + u[t]
                residual[t] += s @ self.w_out.T
            if writes_cache:
                state[slot] = s


class ToyConfig:
    """An architecture of the test's own: layers alternate the toy mixer and attention."""

    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def model_spec(self):
        from ithaca_b200.config import BlockSpec, ModelSpec, PartSpec, default_schedule
        d = self.d
        h, ff = d["hidden_size"], d["intermediate_size"]
        layers = []
        for i in range(d["num_hidden_layers"]):
            p = f"layers.{i}"
            if i % 2 == 0:
                mixer = PartSpec("toy_decay", {"hidden_size": h, "state_size": d["state_size"], "decay": d["decay"]},
                                 {"in": f"{p}.mix.in", "out": f"{p}.mix.out"})
                position = None
            else:
                mixer = PartSpec("attention", {"hidden_size": h, "n_heads": 4, "n_kv_heads": 2, "head_dim": 16,
                                               "window": None, "scale": None},
                                 {k: f"{p}.attn.{k}" for k in ("q", "k", "v", "o")})
                position = PartSpec("rotary", {"rotary_dim": 16, "theta": 10000.0, "pairing": "interleaved", "scaling": None})
            layers.append(BlockSpec("prenorm", mixer,
                                    PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": ff, "activation": "silu"},
                                             {"gate": f"{p}.ff.g", "up": f"{p}.ff.u", "down": f"{p}.ff.d"}),
                                    {"mixer": PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": f"{p}.n1"}),
                                     "feed_forward": PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": f"{p}.n2"})},
                                    position))
        return ModelSpec("ToyDecayLM", d["vocab_size"], h,
                         PartSpec("embedding", {"vocab_size": d["vocab_size"], "hidden_size": h, "scale": 1.0}, {"weight": "emb"}),
                         tuple(layers), default_schedule(len(layers)),
                         PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": "norm"}),
                         PartSpec("lm_head", {"vocab_size": d["vocab_size"], "hidden_size": h, "tied": True}, {"weight": "emb"}),
                         max_position=512)


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from ithaca_b200 import Engine, register_architecture, write_random_model
    from ithaca_b200.config import unregister_architecture
    from ithaca_b200.parts import MIXERS, register_mixer
    register_mixer("toy_decay", ToyDecayMixer)
    register_architecture("ToyDecayLM", ToyConfig)
    try:
        cfg = {"architectures": ["ToyDecayLM"], "hidden_size": 64, "intermediate_size": 96, "num_hidden_layers": 3,
               "vocab_size": 120, "state_size": 24, "decay": 0.9, "torch_dtype": "float32"}
        d = write_random_model(str(tmp_path / "toy"), cfg, seed=2)
        eng = Engine(d, dtype="float32", max_tokens=1024)
        assert [g.name for g in eng.cache.state_groups] == ["decay_state"] and len(eng.cache.kv_groups) == 1
        assert eng.cache.state_groups[0].cache_entries == (0, 2) and eng.cache.kv_groups[0].cache_entries == (1,)
        a, b = random_ids(50, 120, 1), random_ids(23, 120, 2)
        # whole, alone
        s = eng.alloc_slot()
        whole_a = eng.step([s], [a], "all").cpu().numpy()
        eng.free_slot(s)
        s = eng.alloc_slot()                                           # the slot is used again: its state must be zero
        whole_b = eng.step([s], [b], "all").cpu().numpy()
        eng.free_slot(s)
        # together, in pieces: state and keys must be carried per slot
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        rows_a, rows_b = [], []
        lg = eng.step([sa, sb], [a[:20], b[:7]], "all").cpu().numpy()
        rows_a.append(lg[:20]); rows_b.append(lg[20:])
        for t in range(16):
            lg = eng.step([sb, sa], [[b[7 + t]], [a[20 + t]]], "last").cpu().numpy()
            rows_b.append(lg[:1]); rows_a.append(lg[1:])
        eng.free_slot(sb)
        rows_a.append(eng.step([sa], [a[36:]], "all").cpu().numpy())
        assert rel_err(np.concatenate(rows_a), whole_a) <= 2e-5
        assert rel_err(np.concatenate(rows_b), whole_b) <= 2e-5
        # and it generates through the same entry point
        out = eng.generate([a[:5], b[:9]], max_tokens=4, temp=0.0, rep_pen=1.0, stop_token_ids=[])
        assert [len(o) for o in out] == [4, 4]
    finally:
        MIXERS.unregister("toy_decay")
        unregister_architecture("ToyDecayLM")


# ------------------------------------------------------------------------------------------ a toy routed feed-forward and a toy position encoding
class ToySinusoid:
    """A position encoding of the test's own: enc(pos)[2i] = sin(pos / base^(2i/d)), [2i+1] = cos(...), added to
    a mixer's input by the mixer that asks for it.  No weights."""

    @classmethod
    def manifest(cls, spec):
        return {}

    def __init__(self, spec, tensors, runtime):
        self.size, self.base = spec["size"], spec["base"]
        i = torch.arange(0, self.size, 2, dtype=torch.float32, device=runtime.device)
        self.inv = self.base ** (-i / self.size)

    def encode(self, token_pos):
        ang = token_pos.float()[:, None] * self.inv[None, :]
        return torch.stack((torch.sin(ang), torch.cos(ang)), dim=-1).reshape(token_pos.numel(), self.size)


class ToyPositionalMixer:
    """y_t = W (x_t + enc(pos_t)): a mixer without memory that consumes the block's position part."""

    @classmethod
    def manifest(cls, spec):
        from ithaca_b200.weights import TensorReq
        return {spec.weights["w"]: TensorReq((spec["hidden_size"], spec["hidden_size"]))}

    def __init__(self, spec, tensors, runtime, position=None):
        self.w = tensors[spec.weights["w"]].to(runtime.device).float()
        self.position = position

    def cache_requests(self):
        return []

    def forward(self, x, ctx, cache, residual, writes_cache=True):
        residual += (x.float() + self.position.encode(ctx.token_pos)) @ self.w.T


class ToyRoutedFF:
    """Top-1 routing over small experts: e = argmax(router x) (float32 logits, lowest index on ties),
    y = softmax(router x)[e] * W2[e] relu(W1[e] x), added to the residual rows."""

    @classmethod
    def manifest(cls, spec):
        from ithaca_b200.weights import TensorReq
        d, f, E = spec["hidden_size"], spec["expert_size"], spec["n_experts"]
        w = spec.weights
        return {w["router"]: TensorReq((E, d)), w["w1"]: TensorReq((E * f, d)), w["w2"]: TensorReq((E * d, f))}

    def __init__(self, spec, tensors, runtime):
        self.d, self.f, self.E = spec["hidden_size"], spec["expert_size"], spec["n_experts"]
        w = spec.weights
        dev = runtime.device
        self.router = tensors[w["router"]].to(dev).float()
        self.w1 = tensors[w["w1"]].to(dev).float().view(self.E, self.f, self.d)
        self.w2 = tensors[w["w2"]].to(dev).float().view(self.E, self.d, self.f)

    def forward(self, x, ctx, residual):
        x = x.float()
        p = torch.softmax(x @ self.router.T, dim=-1)
        e = torch.argmax(p, dim=-1)
        h = torch.relu(torch.einsum("tfd,td->tf", self.w1[e], x))
        residual += p.gather(1, e[:, None]) * torch.einsum("tdf,tf->td", self.w2[e], h)


class ToyRoutedConfig:
    def __init__(self, d):
        self.d = d

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def model_spec(self):
        from ithaca_b200.config import BlockSpec, ModelSpec, PartSpec, default_schedule
        d = self.d
        h = d["hidden_size"]
        layers = []
        for i in range(d["num_hidden_layers"]):
            p = f"layers.{i}"
            layers.append(BlockSpec(
                "prenorm", PartSpec("toy_positional", {"hidden_size": h}, {"w": f"{p}.mix.w"}),
                PartSpec("toy_routed", {"hidden_size": h, "expert_size": d["expert_size"], "n_experts": d["n_experts"]},
                         {"router": f"{p}.ff.router", "w1": f"{p}.ff.w1", "w2": f"{p}.ff.w2"}),
                {"mixer": PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": f"{p}.n1"}),
                 "feed_forward": PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": f"{p}.n2"})},
                PartSpec("toy_sinusoid", {"size": h, "base": d["base"]})))
        return ModelSpec("ToyRoutedLM", d["vocab_size"], h,
                         PartSpec("embedding", {"vocab_size": d["vocab_size"], "hidden_size": h, "scale": 1.0}, {"weight": "emb"}),
                         tuple(layers), default_schedule(len(layers)),
                         PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": "norm"}),
                         PartSpec("lm_head", {"vocab_size": d["vocab_size"], "hidden_size": h, "tied": False}, {"weight": "head"}),
                         max_position=512)


def toy_routed_plain(cfg, tensors, ids):
    """The same model, whole sequence, float64, written out here."""
    t = {k: v.double() for k, v in tensors.items()}
    h, E, f = cfg["hidden_size"], cfg["n_experts"], cfg["expert_size"]
    x = t["emb"][torch.tensor(ids)]
    pos = torch.arange(len(ids), dtype=torch.float64)
    i = torch.arange(0, h, 2, dtype=torch.float64)
    ang = pos[:, None] * (cfg["base"] ** (-i / h)).float().double()[None, :]
    enc = torch.stack((torch.sin(ang), torch.cos(ang)), dim=-1).reshape(len(ids), h)
    for l in range(cfg["num_hidden_layers"]):
        p = f"layers.{l}"
        x = x + (P.rmsnorm(x, t[f"{p}.n1"], 1e-5) + enc) @ t[f"{p}.mix.w"].T
        xn = P.rmsnorm(x, t[f"{p}.n2"], 1e-5)
        pr = torch.softmax(xn @ t[f"{p}.ff.router"].T, dim=-1)
        e = torch.argmax(pr, dim=-1)
        w1, w2 = t[f"{p}.ff.w1"].view(E, f, h), t[f"{p}.ff.w2"].view(E, h, f)
        hid = torch.relu(torch.einsum("tfd,td->tf", w1[e], xn))
        x = x + pr.gather(1, e[:, None]) * torch.einsum("tdf,tf->td", w2[e], hid)
    return (P.rmsnorm(x, t["norm"], 1e-5) @ t["head"].T).numpy()


def test_a_toy_routed_feed_forward_and_position_encoding_are_registered_built_and_stepped(tmp_path):
    """A feed-forward with routing and a position encoding, both defined here, in an architecture defined here:
    registered, written as a random model folder, loaded, stepped whole and in pieces in a batch, against the same
    model written out plainly.  No file of the framework changes."""
    from ithaca_b200 import Engine, register_architecture, write_random_model
    from ithaca_b200.config import unregister_architecture
    from ithaca_b200.parts import FEED_FORWARDS, MIXERS, POSITIONS, register_feed_forward, register_mixer, register_position
    from ithaca_b200.weights import read_model_tensors
    register_mixer("toy_positional", ToyPositionalMixer)
    register_feed_forward("toy_routed", ToyRoutedFF)
    register_position("toy_sinusoid", ToySinusoid)
    register_architecture("ToyRoutedLM", ToyRoutedConfig)
    try:
        cfg = {"architectures": ["ToyRoutedLM"], "hidden_size": 40, "num_hidden_layers": 2, "vocab_size": 77, "n_experts": 3,
               "expert_size": 24, "base": 50.0, "torch_dtype": "float32"}
        d = write_random_model(str(tmp_path / "toy_routed"), cfg, seed=4)
        eng = Engine(d, dtype="float32", max_tokens=512)
        assert len(eng.cache.kv_groups) == 0 and len(eng.cache.state_groups) == 0
        tensors = read_model_tensors(d)
        a, b = random_ids(30, 77, 5), random_ids(11, 77, 6)
        ref_a, ref_b = toy_routed_plain(cfg, tensors, a), toy_routed_plain(cfg, tensors, b)
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        rows_a, rows_b = [], []
        lg = eng.step([sa, sb], [a[:12], b[:4]], "all").cpu().numpy()
        rows_a.append(lg[:12]); rows_b.append(lg[12:])
        for t in range(7):
            lg = eng.step([sa, sb], [[a[12 + t]], [b[4 + t]]], "last").cpu().numpy()
            rows_a.append(lg[:1]); rows_b.append(lg[1:])
        eng.free_slot(sb)
        rows_a.append(eng.step([sa], [a[19:]], "all").cpu().numpy())
        assert rel_err(np.concatenate(rows_a), ref_a) <= 2e-5
        assert rel_err(np.concatenate(rows_b), ref_b) <= 2e-5
        out = eng.generate([a[:5], b[:9]], max_tokens=3, temp=0.0, rep_pen=1.0, stop_token_ids=[])
        assert [len(o) for o in out] == [3, 3]
    finally:
        MIXERS.unregister("toy_positional")
        FEED_FORWARDS.unregister("toy_routed")
        POSITIONS.unregister("toy_sinusoid")
        unregister_architecture("ToyRoutedLM")
