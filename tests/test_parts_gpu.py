"""Each part alone against the plain functions, and the generality of the assembly: a toy
architecture, defined here, with a mixer that keeps per-sequence state of its own, a block that
runs twice, and a layer that reads another layer's keys and values, registered, built and
stepped without touching the framework's files."""
import dataclasses
import math
from typing import ClassVar

import pytest
import torch

import plain_falcon as plain
import tiny_models as tm

pytestmark = pytest.mark.gpu


def build_ctx(dtype=torch.float32):
    from pytorch_transformers_b200 import kernels
    from pytorch_transformers_b200.parts import BuildContext
    return BuildContext(torch.device("cuda"), dtype, kernels)


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale)


# ------------------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from pytorch_transformers_b200.parts import PartSpec, make_part
    part = make_part(build_ctx(dtype), PartSpec("norm", "layernorm", {"size": 100, "eps": 1e-4}))
    assert set(part.param_decls()) == {"weight", "bias"} and part.param_decls()["weight"].role == "vector"
    g, b, x = rnd(100, seed=1) + 1, rnd(100, seed=2), rnd(7, 100, seed=3).to(dtype)
    part.bind({"weight": g.cuda(), "bias": b.cuda()})
    ref = plain.layer_norm(x.double(), g.double(), b.double(), 1e-4)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(part.forward(x.cuda()).double().cpu(), ref, **tol)


def test_position_parts():
    from pytorch_transformers_b200.parts import PartSpec, make_part
    rot = make_part(build_ctx(), PartSpec("position", "rotary", {"head_dim": 32, "theta": 500042.0, "factor": 2.0}))
    c = {"hidden_size": 64, "num_attention_heads": 2, "rope_theta": 500042.0,
         "rope_scaling": {"rope_type": "linear", "factor": 2.0}}
    assert torch.equal(rot.rotation().cpu(), plain.rope_inv_freq(c)) and rot.score_bias() is None
    for heads in (4, 6, 8, 71):
        ali = make_part(build_ctx(), PartSpec("position", "alibi", {"heads": heads}))
        assert torch.equal(ali.score_bias().cpu(), plain.alibi_slopes(heads).bfloat16().float())
        assert ali.rotation() is None
    with pytest.raises(ValueError):
        make_part(build_ctx(), PartSpec("position", "rotary", {"head_dim": 32, "theta": 1e4, "rotary_dim": 34}))
    with pytest.raises(ValueError, match="no position part of kind 'learned'"):
        make_part(build_ctx(), PartSpec("position", "learned", {}))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act,bias", [("gelu", True), ("gelu_new", False), ("relu", True)])
def test_feed_forward_part(dtype, act, bias):
    from pytorch_transformers_b200.parts import PartSpec, make_part
    part = make_part(build_ctx(dtype), PartSpec("feed_forward", "dense",
                                                {"hidden": 72, "inner": 200, "activation": act, "bias": bias}))
    w = {"up.weight": rnd(200, 72, seed=1, scale=0.1), "down.weight": rnd(72, 200, seed=2, scale=0.1)}
    if bias:
        w.update({"up.bias": rnd(200, seed=3, scale=0.1), "down.bias": rnd(72, seed=4, scale=0.1)})
    assert set(part.param_decls()) == set(w)
    dev = {k: v.to(dtype if k.endswith("weight") else torch.float32).cuda() for k, v in w.items()}
    part.bind(dev)
    x = rnd(9, 72, seed=5).to(dtype)
    wd = {k: (v.to(dtype) if k.endswith("weight") else v).double() for k, v in w.items()}
    u = plain.activation(plain.linear(x.double(), wd["up.weight"], wd.get("up.bias")), act)
    ref = plain.linear(u, wd["down.weight"], wd.get("down.bias"))
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(part.forward(x.cuda(), None).double().cpu(), ref, **tol)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixer_and_block_alone(name, tmp_path):
    """One block of each tiny model, fed a random hidden state, against plain.decoder_layer."""
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts import ScheduleEntry
    folder = tm.tiny_folder(str(tmp_path), name)
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype="float32")
    cfg, w = plain.load_folder(folder, torch.float64)
    c = plain.resolve(cfg)
    lens = [19, 70]
    x = [rnd(n, c["hidden_size"], seed=n) for n in lens]
    cache = model.new_cache(256)
    slots = [cache.open() for _ in lens]
    ctx = StepContext(cache, slots, [[0] * n for n in lens], c["vocab_size"], [[] for _ in lens], model.planners)
    layer = 1
    entry = ScheduleEntry(block=layer, cache_entry=layer)
    block = model.blocks[layer]
    xin = torch.cat(x).cuda()
    from pytorch_transformers_b200.parts import resolve
    got = resolve(model.build.kernels, block.forward(xin, ctx, entry)).double().cpu()   # a block may leave its last sum open
    ref = torch.cat([plain.decoder_layer(t.double(), w, layer, c) for t in x])
    torch.testing.assert_close(got, ref, atol=1e-5, rtol=1e-5)
    # the mixer alone, on the block's normed input
    p = f"transformer.h.{layer}."
    norm_name = "ln_attn" if c["new_decoder_architecture"] and c["num_ln_in_parallel_attn"] == 2 else "input_layernorm"
    a = [plain.layer_norm(t.double(), w[p + norm_name + ".weight"], w[p + norm_name + ".bias"],
                          c["layer_norm_epsilon"]) for t in x]
    got_attn = block.mixer.forward(torch.cat(a).float().cuda(), ctx, entry).double().cpu()
    ref_attn = torch.cat([plain.self_attention(t, w, p + "self_attention.", c) for t in a])
    torch.testing.assert_close(got_attn, ref_attn, atol=1e-5, rtol=1e-5)


# ------------------------------------------------------------------------------ a toy architecture
def _register_toy():
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.base import ModelConfig
    from pytorch_transformers_b200.parts import (ModelSpec, ParamDecl, Part, PartSpec, ScheduleEntry, StateNeed,
                                                 register_part)

    @register_part("mixer", "toy_running_mean")
    class RunningMean(Part):
        """y_t = W mean(x_0 .. x_t): per-sequence state = (sum of inputs, count). Torch ops: a toy."""

        def __init__(self, build, spec, hidden):
            super().__init__(build, spec)
            self.hidden = hidden
            self.p_w_weight = None

        def param_decls(self):
            return {"w.weight": ParamDecl((self.hidden, self.hidden))}

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed(self.hidden + 1)

        def forward(self, x, ctx, entry):
            state = ctx.cache.entry_state(entry.cache_entry)
            out = torch.empty_like(x)
            start = 0
            for slot, n in zip(ctx.slots, ctx.new):
                st = state[slot]
                sums = st[:-1][None, :] + torch.cumsum(x[start:start + n].float(), 0)
                counts = st[-1] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[start:start + n] = ((sums / counts[:, None]) @ self.p_w_weight.float().T).to(x.dtype)
                st[:-1] = sums[-1]
                st[-1] = counts[-1]
                start += n
            return out

    @dataclasses.dataclass
    class ToyConfig(ModelConfig):
        model_type: ClassVar[str] = "toy_mix"
        vocab_size: int = 50
        hidden_size: int = 32
        heads: int = 4
        kv_heads: int = 2

    def block(cfg, i, mixer):
        p = f"blocks.{i}."
        norm = PartSpec("norm", "rmsnorm", {"size": cfg.hidden_size, "eps": 1e-5}, names={"weight": p + "norm.weight"})
        ff = PartSpec("feed_forward", "dense", {"hidden": cfg.hidden_size, "inner": 48, "activation": "relu"},
                      names={"up.weight": p + "ff.up.weight", "down.weight": p + "ff.down.weight"})
        return PartSpec("block", "parallel", children={"norm_mixer": norm, "mixer": mixer, "feed_forward": ff})

    def spec(cfg):
        d = cfg.hidden_size // cfg.heads

        def attn(i):
            return PartSpec("mixer", "attention", {"hidden": cfg.hidden_size, "heads": cfg.heads,
                                                   "kv_heads": cfg.kv_heads, "head_dim": d},
                            children={"position": PartSpec("position", "rotary", {"head_dim": d, "theta": 100.0})},
                            names={"qkv.weight": f"blocks.{i}.attn.qkv.weight", "out.weight": f"blocks.{i}.attn.out.weight"})

        blocks = [block(cfg, 0, attn(0)),
                  block(cfg, 1, PartSpec("mixer", "toy_running_mean", {"hidden": cfg.hidden_size},
                                         names={"w.weight": "blocks.1.mix.w.weight"})),
                  block(cfg, 2, attn(2))]
        # block 0 runs twice (two cache entries); block 2 reads block 0's first cache entry
        schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(2, 0, writes_cache=False)]
        return ModelSpec(cfg.vocab_size, cfg.hidden_size, "embed.weight", blocks,
                         PartSpec("norm", "rmsnorm", {"size": cfg.hidden_size, "eps": 1e-5},
                                  names={"weight": "final_norm.weight"}), None, schedule)

    ptb.register_architecture("toy_mix", ("ToyMixForCausalLM",), ToyConfig, spec)
    return ToyConfig


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer_repeated_block_and_shared_cache(tmp_path, dtype):
    import pytorch_transformers_b200 as ptb
    ToyConfig = _register_toy()
    # bfloat16 with head size 64: single-token steps run the one-kernel decode attention, also for the
    # block that reads another block's cache entry
    cfg = ToyConfig() if dtype == "float32" else ToyConfig(hidden_size=256)
    folder = ptb.write_random_model(cfg, seed=3, folder=str(tmp_path / "toy"), dtype=getattr(torch, dtype))
    assert ptb.AutoConfig.from_pretrained(folder) == cfg
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    cache = model.new_cache(512)
    assert len(cache.groups) == 1 and cache.groups[0].entries == [0, 2]      # entries 0 and 2 hold K/V
    assert cache.state_width == cfg.hidden_size + 1 and cache.entry_state(1) is not None
    g = torch.Generator().manual_seed(0)
    reqs = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (70, 9, 33)]
    whole = []
    for ids in reqs:
        s = cache.open()
        whole.append(model.step(cache, [s], [ids], want="all"))
        cache.close(s)
    # token by token, batched with unequal lengths, on reused slots (state must have been zeroed)
    slots = [cache.open() for _ in reqs]
    heads = [5, 2, 33 - 8]
    out = model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="last")
    live = list(range(3))
    t = 0
    while live:
        for i in live:
            row = live.index(i)
            torch.testing.assert_close(out[row], whole[i][heads[i] + t - 1], **tol)
        live = [i for i in live if heads[i] + t < len(reqs[i])]
        if not live:
            break
        out = model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
        t += 1
    # and against a plain computation of the same toy model
    _, w = plain.load_folder(folder, torch.float64)
    ref = toy_plain(reqs[0], w, cfg)
    torch.testing.assert_close(whole[0].double().cpu(), ref, **tol)
    # token by token the same: the last block reads the first block's cache entry in every step
    # generation works on it as on any model
    gen = model.generate([reqs[1]], max_new_tokens=4, eos_token_id=None)
    assert len(gen[0]) == len(reqs[1]) + 4


def toy_plain(ids, w, cfg):
    d = cfg.hidden_size // cfg.heads
    c = {"num_attention_heads": cfg.heads, "hidden_size": cfg.hidden_size, "new_decoder_architecture": True,
         "num_kv_heads": cfg.kv_heads, "rope_theta": 100.0, "rope_scaling": None}

    def rms(x, g):
        return x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-5) * g

    def ff(x, i):
        return torch.relu(x @ w[f"blocks.{i}.ff.up.weight"].T) @ w[f"blocks.{i}.ff.down.weight"].T

    def attn(a, i, kv=None):
        q, k, v = plain.split_heads(a @ w[f"blocks.{i}.attn.qkv.weight"].T, c)
        pos = torch.arange(a.shape[0])
        inv = plain.rope_inv_freq(c)
        q, k = plain.rotary(q, pos, inv), plain.rotary(k, pos, inv)
        if kv is not None:
            k, v = kv
        return plain.attention_core(q, k, v, c) @ w[f"blocks.{i}.attn.out.weight"].T, (k, v)

    x = w["embed.weight"][torch.tensor(ids)]
    a = rms(x, w["blocks.0.norm.weight"])
    y, kv0 = attn(a, 0)
    x = x + (ff(a, 0) + y)
    a = rms(x, w["blocks.1.norm.weight"])
    mean = torch.cumsum(a, 0) / torch.arange(1, len(ids) + 1, dtype=a.dtype)[:, None]
    x = x + (ff(a, 1) + mean @ w["blocks.1.mix.w.weight"].T)
    a = rms(x, w["blocks.0.norm.weight"])
    y, _ = attn(a, 0)
    x = x + (ff(a, 0) + y)
    a = rms(x, w["blocks.2.norm.weight"])
    y, _ = attn(a, 2, kv=kv0)
    x = x + (ff(a, 2) + y)
    return rms(x, w["final_norm.weight"]) @ w["embed.weight"].T


# ------------------------------------------ a second toy: routed feed-forward, other position encodings
def _register_toy_routed():
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.base import ModelConfig
    from pytorch_transformers_b200.parts import ModelSpec, ParamDecl, Part, PartSpec, ScheduleEntry, register_part

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(Part):
        """Router logits in float32, the best expert per token, that expert's relu MLP scaled by its
        softmax weight. Torch ops: a toy that shows the interface (forward(x, ctx) -> [tokens, hidden])."""

        def __init__(self, build, spec, hidden, inner, experts):
            super().__init__(build, spec)
            self.hidden, self.inner, self.experts = hidden, inner, experts

        def param_decls(self):
            d = {"router.weight": ParamDecl((self.experts, self.hidden))}
            for e in range(self.experts):
                d[f"experts.{e}.up.weight"] = ParamDecl((self.inner, self.hidden))
                d[f"experts.{e}.down.weight"] = ParamDecl((self.hidden, self.inner))
            return d

        def forward(self, x, ctx):
            logits = x.float() @ self.p_router_weight.float().T
            gate, pick = torch.softmax(logits, -1).max(-1)
            out = torch.zeros_like(x, dtype=torch.float32)
            for e in range(self.experts):
                rows = (pick == e).nonzero().flatten()
                if rows.numel():
                    up = getattr(self, f"p_experts_{e}_up_weight").float()
                    down = getattr(self, f"p_experts_{e}_down_weight").float()
                    out[rows] = torch.relu(x[rows].float() @ up.T) @ down.T * gate[rows, None]
            return out.to(x.dtype)

    @register_part("position", "toy_two_speed")
    class TwoSpeedRotation(Part):
        """Rotation whose first half of the pairs turns fast and whose second half turns slowly."""

        def __init__(self, build, spec, head_dim):
            super().__init__(build, spec)
            half = head_dim // 2
            self.inv_freq = torch.cat([torch.full((half - half // 2,), 0.5), torch.full((half // 2,), 0.01)]).to(build.device)

        def rotation(self):
            return self.inv_freq

        def score_bias(self):
            return None

    @register_part("position", "toy_head_decay")
    class HeadDecay(Part):
        """A per-head slope times the key's position added to the scores (the interface ALiBi uses)."""

        def __init__(self, build, spec, heads):
            super().__init__(build, spec)
            self.slopes = (0.25 / torch.arange(1, heads + 1, dtype=torch.float32)).bfloat16().float().to(build.device)

        def rotation(self):
            return None

        def score_bias(self):
            return self.slopes

    @dataclasses.dataclass
    class ToyRoutedConfig(ModelConfig):
        model_type: ClassVar[str] = "toy_routed"
        vocab_size: int = 61
        hidden_size: int = 48
        heads: int = 3
        experts: int = 3

    def spec(cfg):
        d = cfg.hidden_size // cfg.heads
        h = cfg.hidden_size

        def norm(name):
            return PartSpec("norm", "layernorm", {"size": h, "eps": 1e-5}, names={"weight": name + ".weight", "bias": name + ".bias"})

        def attn(i, position):
            return PartSpec("mixer", "attention", {"hidden": h, "heads": cfg.heads, "kv_heads": 1, "head_dim": d},
                            children={"position": position},
                            names={"qkv.weight": f"l{i}.attn.qkv.weight", "out.weight": f"l{i}.attn.out.weight"})

        dense = PartSpec("feed_forward", "dense", {"hidden": h, "inner": 80, "activation": "gelu"},
                         names={"up.weight": "l0.ff.up.weight", "down.weight": "l0.ff.down.weight"})
        routed_names = {"router.weight": "l1.moe.router.weight"}
        for e in range(cfg.experts):
            routed_names[f"experts.{e}.up.weight"] = f"l1.moe.experts.{e}.up.weight"
            routed_names[f"experts.{e}.down.weight"] = f"l1.moe.experts.{e}.down.weight"
        routed = PartSpec("feed_forward", "toy_top1_experts", {"hidden": h, "inner": 40, "experts": cfg.experts},
                          names=routed_names)
        blocks = [PartSpec("block", "sequential", children={
                      "norm_mixer": norm("l0.ln1"), "norm_ff": norm("l0.ln2"),
                      "mixer": attn(0, PartSpec("position", "toy_two_speed", {"head_dim": d})), "feed_forward": dense}),
                  PartSpec("block", "sequential", children={
                      "norm_mixer": norm("l1.ln1"), "norm_ff": norm("l1.ln2"),
                      "mixer": attn(1, PartSpec("position", "toy_head_decay", {"heads": cfg.heads})),
                      "feed_forward": routed})]
        return ModelSpec(cfg.vocab_size, h, "embed.weight", blocks, norm("ln_f"), "head.weight",
                         [ScheduleEntry(0, 0), ScheduleEntry(1, 1)])

    ptb.register_architecture("toy_routed", ("ToyRoutedForCausalLM",), ToyRoutedConfig, spec)
    return ToyRoutedConfig


def toy_routed_plain(ids, w, cfg):
    h, nh = cfg.hidden_size, cfg.heads
    d = h // nh
    c = {"num_attention_heads": nh, "hidden_size": h, "new_decoder_architecture": False, "multi_query": True,
         "num_kv_heads": 1}

    def ln(x, name):
        return plain.layer_norm(x, w[name + ".weight"], w[name + ".bias"], 1e-5)

    def attn(a, i, inv=None, slopes=None):
        q, k, v = plain.split_heads(a @ w[f"l{i}.attn.qkv.weight"].T, c)
        pos = torch.arange(a.shape[0])
        bias = None
        if inv is not None:
            q, k = plain.rotary(q, pos, inv), plain.rotary(k, pos, inv)
        if slopes is not None:
            bias = (slopes[:, None].bfloat16() * pos[None, :]).to(a.dtype)     # the product in bfloat16, as for ALiBi
        return plain.attention_core(q, k, v, c, bias) @ w[f"l{i}.attn.out.weight"].T

    half = d // 2
    inv = torch.cat([torch.full((half - half // 2,), 0.5), torch.full((half // 2,), 0.01)])
    slopes = 0.25 / torch.arange(1, nh + 1, dtype=torch.float32)
    x = w["embed.weight"][torch.tensor(ids)]
    x = x + attn(ln(x, "l0.ln1"), 0, inv=inv)
    m = ln(x, "l0.ln2")
    x = x + plain.activation(m @ w["l0.ff.up.weight"].T, "gelu") @ w["l0.ff.down.weight"].T
    x = x + attn(ln(x, "l1.ln1"), 1, slopes=slopes)
    m = ln(x, "l1.ln2")
    gate, pick = torch.softmax(m.float() @ w["l1.moe.router.weight"].float().T, -1).max(-1)
    moe = torch.zeros_like(m)
    for t in range(m.shape[0]):
        e = int(pick[t])
        moe[t] = torch.relu(m[t] @ w[f"l1.moe.experts.{e}.up.weight"].T) @ w[f"l1.moe.experts.{e}.down.weight"].T * gate[t]
    x = x + moe
    return ln(x, "ln_f") @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_routed_feed_forward_and_other_position_encodings(tmp_path, dtype):
    """Parts defined here (a feed-forward that routes each token to one of three experts, a rotation
    with its own frequencies, a per-head score slope) are registered, built from a specification
    that gives each layer its own mixer and feed-forward, loaded from a folder of random weights and
    stepped: whole prompts, batches of unequal lengths, token by token. No file of the framework knows them."""
    import pytorch_transformers_b200 as ptb
    Config = _register_toy_routed()
    cfg = Config()
    tdtype = getattr(torch, dtype)
    folder = ptb.write_random_model(cfg, seed=5, folder=str(tmp_path / "toy_routed"), dtype=tdtype)
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    _, w = plain.load_folder(folder, torch.float64)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    g = torch.Generator().manual_seed(1)
    reqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (67, 5, 130)]
    refs = [toy_routed_plain(ids, w, cfg) for ids in reqs]
    cache = model.new_cache(512)
    slots = [cache.open() for _ in reqs]
    heads = [60, 3, 130 - 20]
    out = model.step(cache, slots, [r[:n] for r, n in zip(reqs, heads)], want="last")
    live, t, routed_differently = list(range(3)), 0, 0
    while live:
        for row, i in enumerate(live):
            got, ref = out[row].double().cpu(), refs[i][heads[i] + t - 1]
            if dtype == "bfloat16" and not torch.allclose(got, ref, **tol):
                routed_differently += 1     # a near-tie of two experts may fall the other way in bfloat16
                continue
            torch.testing.assert_close(got, ref, **tol)
        live = [i for i in live if heads[i] + t < len(reqs[i])]
        if not live:
            break
        out = model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
        t += 1
    assert routed_differently <= 2
    cache.close_all()
    cache.check()
    gen = model.generate([reqs[1]], max_new_tokens=3, eos_token_id=None)
    assert len(gen[0]) == len(reqs[1]) + 3


# ------------------------------------------------ a third toy: a layer with all keys and a layer with a window
def _register_toy_window():
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.base import ModelConfig
    from pytorch_transformers_b200.parts import ModelSpec, PartSpec, ScheduleEntry

    @dataclasses.dataclass
    class ToyWindowConfig(ModelConfig):
        model_type: ClassVar[str] = "toy_window"
        vocab_size: int = 97
        hidden_size: int = 128
        heads: int = 2
        window: int = 40

    def spec(cfg):
        h, d = cfg.hidden_size, cfg.hidden_size // cfg.heads

        def norm(name):
            return PartSpec("norm", "rmsnorm", {"size": h, "eps": 1e-6}, names={"weight": name + ".weight"})

        def block(i, window):
            attn = PartSpec("mixer", "attention", {"hidden": h, "heads": cfg.heads, "kv_heads": 1, "head_dim": d,
                                                   "window": window},
                            children={"position": PartSpec("position", "rotary", {"head_dim": d, "theta": 1000.0})},
                            names={"qkv.weight": f"l{i}.qkv.weight", "out.weight": f"l{i}.out.weight"})
            ff = PartSpec("feed_forward", "dense", {"hidden": h, "inner": 96, "activation": "relu"},
                          names={"up.weight": f"l{i}.up.weight", "down.weight": f"l{i}.down.weight"})
            return PartSpec("block", "sequential", children={"norm_mixer": norm(f"l{i}.n1"), "norm_ff": norm(f"l{i}.n2"),
                                                             "mixer": attn, "feed_forward": ff})

        return ModelSpec(cfg.vocab_size, h, "embed.weight", [block(0, 0), block(1, cfg.window)], norm("nf"), None,
                         [ScheduleEntry(0, 0), ScheduleEntry(1, 1)])

    ptb.register_architecture("toy_window", ("ToyWindowForCausalLM",), ToyWindowConfig, spec)
    return ToyWindowConfig


def toy_window_plain(ids, w, cfg):
    h, nh = cfg.hidden_size, cfg.heads
    d = h // nh
    c = {"num_attention_heads": nh, "hidden_size": h, "new_decoder_architecture": False, "multi_query": True,
         "num_kv_heads": 1}
    inv = 1.0 / (1000.0 ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))

    def rms(x, name):
        return x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-6) * w[name + ".weight"]

    def attn(a, i, window):
        q, k, v = plain.split_heads(a @ w[f"l{i}.qkv.weight"].T, c)
        pos = torch.arange(a.shape[0])
        q, k = plain.rotary(q, pos, inv), plain.rotary(k, pos, inv)
        s = a.shape[0]
        out = torch.empty(s, nh, d, dtype=a.dtype)
        seen = pos[None, :] <= pos[:, None]
        if window:
            seen = seen & (pos[None, :] > pos[:, None] - window)     # the query's own position and window - 1 before it
        for hh in range(nh):
            scores = (q[:, hh] @ k[:, 0].T) / math.sqrt(d)
            out[:, hh] = torch.softmax(scores.masked_fill(~seen, float("-inf")), -1) @ v[:, 0]
        return out.reshape(s, h) @ w[f"l{i}.out.weight"].T

    x = w["embed.weight"][torch.tensor(ids)]
    for i, window in ((0, 0), (1, cfg.window)):
        x = x + attn(rms(x, f"l{i}.n1"), i, window)
        m = rms(x, f"l{i}.n2")
        x = x + torch.relu(m @ w[f"l{i}.up.weight"].T) @ w[f"l{i}.down.weight"].T
    return rms(x, "nf") @ w["embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_full_and_a_windowed_layer(tmp_path, dtype):
    """Two storage groups in one cache: the first layer keeps all keys, the second a window of 40 (no
    multiple of the page), whose pages behind the window go back to the pool while the sequences grow.
    Prompts longer than the window, batches of unequal lengths, 100 single-token steps on a cache that
    would not hold the windowed layer's keys without the release."""
    import pytorch_transformers_b200 as ptb
    Config = _register_toy_window()
    cfg = Config()
    folder = ptb.write_random_model(cfg, seed=9, folder=str(tmp_path / "toy_window"), dtype=getattr(torch, dtype))
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    _, w = plain.load_folder(folder, torch.float64)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    g = torch.Generator().manual_seed(4)
    reqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (230, 45, 131)]
    refs = [toy_window_plain(ids, w, cfg) for ids in reqs]
    cache = model.new_cache(64 * 8)
    kinds = sorted(grp.need.kind for grp in cache.groups)
    assert kinds == ["full", "window"]
    slots = [cache.open() for _ in reqs]
    heads = [130, 5, 31]
    out = model.step(cache, slots, [r[:n] for r, n in zip(reqs, heads)], want="last")
    live, t = list(range(3)), 0
    while live:
        for row, i in enumerate(live):
            torch.testing.assert_close(out[row].double().cpu(), refs[i][heads[i] + t - 1], **tol)
        live = [i for i in live if heads[i] + t < len(reqs[i])]
        if not live:
            break
        out = model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
        t += 1
        window_group = next(grp for grp in cache.groups if grp.need.kind == "window")
        assert window_group.pool.in_use <= 2 * len(live) + 1      # a window of 40 spans at most two pages
    cache.close_all()
    cache.check()


# ------------------------------------------ a stateful mixer whose steps are replayed as CUDA graphs
def _register_toy_graph_state():
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.base import ModelConfig
    from pytorch_transformers_b200.parts import ModelSpec, ParamDecl, Part, PartSpec, StateNeed, register_part

    @register_part("mixer", "toy_decaying_sum")
    class DecayingSum(Part):
        """state <- decay * state + x_t, y_t = W state: per-sequence state, updated through the step's
        device arrays only (slots come from ctx.dev), so steps of single tokens may be captured."""
        graph_safe = True

        def __init__(self, build, spec, hidden, decay):
            super().__init__(build, spec)
            self.hidden, self.decay = hidden, float(decay)

        def param_decls(self):
            return {"w.weight": ParamDecl((self.hidden, self.hidden))}

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed(self.hidden)

        def forward(self, x, ctx, entry):
            state = ctx.cache.entry_state(entry.cache_entry)
            if not ctx.is_decode:
                raise NotImplementedError("the toy takes one token per sequence and step")
            slots = ctx.dev["slots"].long()
            new = state.index_select(0, slots) * self.decay + x.float()
            state.index_copy_(0, slots, new)
            return (new @ self.p_w_weight.float().T).to(x.dtype)

    @dataclasses.dataclass
    class ToyStateConfig(ModelConfig):
        model_type: ClassVar[str] = "toy_graph_state"
        vocab_size: int = 40
        hidden_size: int = 32

    def spec(cfg):
        norm = lambda n: PartSpec("norm", "rmsnorm", {"size": cfg.hidden_size, "eps": 1e-5}, names={"weight": n})
        ff = PartSpec("feed_forward", "dense", {"hidden": cfg.hidden_size, "inner": 48, "activation": "gelu"},
                      names={"up.weight": "b.ff.up.weight", "down.weight": "b.ff.down.weight"})
        mixer = PartSpec("mixer", "toy_decaying_sum", {"hidden": cfg.hidden_size, "decay": 0.5},
                         names={"w.weight": "b.mix.w.weight"})
        block = PartSpec("block", "sequential", children={"norm_mixer": norm("b.n1.weight"), "norm_ff": norm("b.n2.weight"),
                                                          "mixer": mixer, "feed_forward": ff})
        return ModelSpec(cfg.vocab_size, cfg.hidden_size, "embed.weight", [block], norm("final.weight"), None)

    ptb.register_architecture("toy_graph_state", ("ToyGraphState",), ToyStateConfig, spec)
    return ToyStateConfig


def test_a_stateful_mixer_under_graph_replay_updates_its_state_once_per_step():
    """A registered mixer with per-sequence state and graph_safe = True: its single-token steps are
    captured and replayed, the first step of every batch size included, and give what the same model
    gives without graphs (a step that ran twice would have advanced the state twice)."""
    import pytorch_transformers_b200 as ptb
    Cfg = _register_toy_graph_state()
    model = ptb.AutoModelForCausalLM.from_config(Cfg(), seed=5, dtype="float32")
    assert model.use_graphs and not model.planners
    seqs = [[3, 9, 1, 30, 22, 8, 17], [5, 5, 12, 2], [39, 0]]

    def run():
        cache = model.new_cache(64 * 4)
        slots = [cache.open() for _ in seqs]
        outs = []
        for t in range(max(map(len, seqs))):
            live = [i for i, s in enumerate(seqs) if t < len(s)]
            outs.append(model.step(cache, [slots[i] for i in live], [[seqs[i][t]] for i in live]))
        return torch.cat(outs), cache

    with_graphs, cache = run()
    assert len(cache.__dict__.get("_step_graphs", {})) == 3            # batch sizes 3, 2 and 1
    again, _ = run()                                                    # new cache, new graphs, fresh state
    model.use_graphs = False
    without, _ = run()
    assert torch.equal(with_graphs, without) and torch.equal(again, without)
    # and the state is what the recurrence says: s = sum_k 0.5^k x_{t-k}
    model.use_graphs = True
    cache = model.new_cache(64)
    slot = cache.open()
    for tok in seqs[0]:
        model.step(cache, [slot], [[tok]])
    emb = model.embedding[torch.tensor(seqs[0], device="cuda")].float()
    gain = model.blocks[0].children["norm_mixer"].p_weight
    normed = emb / torch.sqrt((emb ** 2).mean(-1, keepdim=True) + 1e-5) * gain
    want = sum(0.5 ** (len(seqs[0]) - 1 - k) * normed[k] for k in range(len(seqs[0])))
    torch.testing.assert_close(cache.entry_state(0)[slot], want, atol=1e-5, rtol=1e-5)


# ------------------------------------------ a toy with a scale and a norm on the embeddings, a scale on the logits
def _register_toy_scaled():
    import pytorch_transformers_b200 as ptb
    from pytorch_transformers_b200.config.base import ModelConfig
    from pytorch_transformers_b200.parts import ModelSpec, PartSpec

    @dataclasses.dataclass
    class ToyScaledConfig(ModelConfig):
        model_type: ClassVar[str] = "toy_scaled"
        vocab_size: int = 60
        hidden_size: int = 48
        heads: int = 3
        interleaved: bool = False       # rotated pairs (2 i, 2 i + 1) instead of (i, i + head_dim / 2)

    def spec(cfg):
        d = cfg.hidden_size // cfg.heads
        ln = lambda n: PartSpec("norm", "layernorm", {"size": cfg.hidden_size, "eps": 1e-5, "bias": True},
                                names={"weight": n + ".weight", "bias": n + ".bias"})
        mixer = PartSpec("mixer", "attention", {"hidden": cfg.hidden_size, "heads": cfg.heads, "kv_heads": 1, "head_dim": d},
                         children={"position": PartSpec("position", "rotary", {"head_dim": d, "theta": 1000.0,
                                                                               "interleaved": cfg.interleaved})},
                         names={"qkv.weight": "b.attn.qkv.weight", "out.weight": "b.attn.out.weight"})
        ff = PartSpec("feed_forward", "dense", {"hidden": cfg.hidden_size, "inner": 64, "activation": "gelu"},
                      names={"up.weight": "b.ff.up.weight", "down.weight": "b.ff.down.weight"})
        block = PartSpec("block", "parallel", children={"norm_mixer": ln("b.ln"), "mixer": mixer, "feed_forward": ff})
        return ModelSpec(cfg.vocab_size, cfg.hidden_size, "embed.weight", [block], ln("final"), None,
                         embedding_scale=math.sqrt(cfg.hidden_size), embedding_norm=ln("embed_ln"), logit_scale=0.25)

    ptb.register_architecture("toy_scaled", ("ToyScaled",), ToyScaledConfig, spec)
    return ToyScaledConfig


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_scaled_and_normed_embeddings_and_scaled_logits(tmp_path, dtype):
    """What some architectures do between the table and the first block and after the head is data of the
    ModelSpec (embedding_scale, embedding_norm, logit_scale), not an edit of the engine."""
    import pytorch_transformers_b200 as ptb
    Cfg = _register_toy_scaled()
    cfg = Cfg()
    folder = ptb.write_random_model(cfg, seed=8, folder=str(tmp_path / "scaled"), dtype=getattr(torch, dtype))
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    assert "embed_ln.weight" in model.param_table() and model.embedding_norm is not None
    _, w = plain.load_folder(folder, torch.float64)
    ids = torch.randint(0, 60, (23,), generator=torch.Generator().manual_seed(1)).tolist()
    c = {"num_attention_heads": 3, "hidden_size": 48, "new_decoder_architecture": False, "multi_query": True,
         "rope_theta": 1000.0, "rope_scaling": None}
    x = w["embed.weight"][torch.tensor(ids)] * math.sqrt(48)
    if dtype == "bfloat16":
        x = x.bfloat16().double()
    x = plain.layer_norm(x, w["embed_ln.weight"], w["embed_ln.bias"], 1e-5)
    a = plain.layer_norm(x, w["b.ln.weight"], w["b.ln.bias"], 1e-5)
    q, k, v = plain.split_heads(a @ w["b.attn.qkv.weight"].T, c)
    pos, inv = torch.arange(len(ids)), plain.rope_inv_freq(c)
    attn = plain.attention_core(plain.rotary(q, pos, inv), plain.rotary(k, pos, inv), v, c) @ w["b.attn.out.weight"].T
    ff = plain.activation(a @ w["b.ff.up.weight"].T, "gelu") @ w["b.ff.down.weight"].T
    x = x + (ff + attn)
    ref = plain.layer_norm(x, w["final.weight"], w["final.bias"], 1e-5) @ w["embed.weight"].T * 0.25
    cache = model.new_cache(64)
    slot = cache.open()
    got = torch.cat([model.step(cache, [slot], [ids[:20]], want="all")] +
                    [model.step(cache, [slot], [[t]]) for t in ids[20:]])
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(got.double().cpu(), ref, **tol)
    model.check_errors()


def _scaled_plain(ids, w, hidden, heads, interleaved, bf16):
    """The toy_scaled model on one whole sequence in float64."""
    c = {"num_attention_heads": heads, "hidden_size": hidden, "new_decoder_architecture": False, "multi_query": True,
         "rope_theta": 1000.0, "rope_scaling": None}

    def rot(x, pos, inv):
        if not interleaved:
            return plain.rotary(x, pos, inv)
        ang = pos.float()[:, None] * inv[None, :]
        cos, sin = ang.cos().double()[:, None, :], ang.sin().double()[:, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = b * cos + a * sin
        return out

    x = w["embed.weight"][torch.tensor(ids)] * math.sqrt(hidden)
    if bf16:
        x = x.bfloat16().double()
    x = plain.layer_norm(x, w["embed_ln.weight"], w["embed_ln.bias"], 1e-5)
    a = plain.layer_norm(x, w["b.ln.weight"], w["b.ln.bias"], 1e-5)
    fused = a @ w["b.attn.qkv.weight"].T
    if bf16:
        fused = fused.bfloat16().double()       # the engine holds the projection, and the rotated q and k, in bfloat16
    q, k, v = plain.split_heads(fused, c)
    pos, inv = torch.arange(len(ids)), plain.rope_inv_freq(c)
    q, k = rot(q, pos, inv), rot(k, pos, inv)
    if bf16:
        q, k = q.bfloat16().double(), k.bfloat16().double()
    attn = plain.attention_core(q, k, v, c) @ w["b.attn.out.weight"].T
    ff = plain.activation(a @ w["b.ff.up.weight"].T, "gelu") @ w["b.ff.down.weight"].T
    x = x + (ff + attn)
    return plain.layer_norm(x, w["final.weight"], w["final.bias"], 1e-5) @ w["embed.weight"].T * 0.25


@pytest.mark.parametrize("dtype,hidden,heads,larger", [("float32", 48, 3, 16.0), ("bfloat16", 2560, 40, 4.0)])
def test_rotation_of_adjacent_pairs(tmp_path, dtype, hidden, heads, larger):
    """A rotary part with ``interleaved=True`` rotates the pairs (2 i, 2 i + 1): in the kernel that splits
    and stores prompts, in the one-kernel decode attention and in the tcgen05 decode attention (40 heads
    of size 64 on one K/V head: steps of 3 and of 50 single tokens)."""
    import pytorch_transformers_b200 as ptb
    Cfg = _register_toy_scaled()
    cfg = Cfg(hidden_size=hidden, heads=heads, interleaved=True)
    folder = ptb.write_random_model(cfg, seed=10, folder=str(tmp_path / "inter"), dtype=getattr(torch, dtype))
    model = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    _, w = plain.load_folder(folder, torch.float64)
    # With weights of 0.02 the scores are all but equal and the rotation could be anything: the fused
    # projection is made larger (by a power of two, exact in both dtypes) on both sides, so that which
    # dims turn together decides which keys a query finds, and the other pairing would miss the
    # tolerance many times over.
    model.blocks[0].children["mixer"].p_qkv_weight.mul_(larger)
    w["b.attn.qkv.weight"] = w["b.attn.qkv.weight"] * larger
    g = torch.Generator().manual_seed(2)
    reqs = [torch.randint(0, 60, (n,), generator=g).tolist() for n in (75, 9, 30)]
    refs = [_scaled_plain(r, w, hidden, heads, True, dtype == "bfloat16") for r in reqs]
    other = _scaled_plain(reqs[0], w, hidden, heads, False, dtype == "bfloat16")
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)
    assert (refs[0] - other).abs().max() > 5 * (tol["atol"] + tol["rtol"] * refs[0].abs().max())
    cache = model.new_cache(64 * 4 + 64 * 50)
    slots = [cache.open() for _ in reqs]
    heads_ = [70, 4, 25]
    out = model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads_)], want="last")
    for t in range(4):
        for row in range(3):
            torch.testing.assert_close(out[row].double().cpu(), refs[row][heads_[row] + t - 1], **tol)
        out = model.step(cache, slots, [[r[h + t]] for r, h in zip(reqs, heads_)])
    if heads == 40:
        many = [cache.open() for _ in range(50)]
        for i in range(0, 50, 10):
            model.step(cache, many[i:i + 10], [reqs[1][:5]] * 10, want="none")
        out = model.step(cache, many, [[reqs[1][5]]] * 50)
        torch.testing.assert_close(out.double().cpu(), refs[1][5][None, :].expand(50, -1), **tol)
    model.check_errors()
