"""Each part of a layer alone against the plain implementation's function for that part, at
sizes other than the tiny models'; and a toy mixer with state of its own, defined here,
that is registered, built into a toy architecture, loaded from a random-weights folder and
stepped through the engine without a change to the framework's files."""
import os
from dataclasses import dataclass
from typing import Any, Dict

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rt(dtype):
    from atom_b200.parts.base import Runtime, Workspace
    return Runtime(dtype, torch.device(DEV), Workspace(torch.device(DEV)))


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * scale


def _bind(part, tensors, rt):
    dev = {}
    for k, v in tensors.items():
        spec = part.params()[k]
        dt = rt.dtype if spec.role == "matrix" else (torch.float32 if rt.dtype == torch.float32 else torch.bfloat16)
        dev[k] = v.to(dt).to(DEV).contiguous()
    part.bind(dev, rt)
    # what the part actually holds, widened: the reference computes on the same values
    return {k: v.double().cpu() for k, v in dev.items()}


def _tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


def _assert_mixer_close(got, want, dtype):
    """32-bit: the order of sums only.  bfloat16: the bounds of tests/test_replay_gpu.py for
    outputs that pass through a sharpened softmax: single elements within 8 % of the largest
    magnitude, the whole within 1 % rms of it."""
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
        return
    scale = float(want.abs().max())
    err = (got - want).abs()
    assert float(err.max()) <= 8e-2 * scale, f"max abs error {float(err.max()):.3e} of scale {scale:.3e}"
    assert float((err ** 2).mean().sqrt()) <= 1e-2 * scale, f"rms error {float((err ** 2).mean().sqrt()):.3e}"


class _Cache:
    """A cache manager, its storage and a step builder for one mixer's need."""

    def __init__(self, need, dtype, page=8, pages=64):
        from atom_b200.cache import CacheManager
        from atom_b200.cache.storage import CacheStorage
        from atom_b200.engine.batch import StepBuilder

        self.manager = CacheManager({0: need}, page, pages, 8)
        self.storage = CacheStorage(self.manager, dtype, torch.device(DEV))
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.builder = StepBuilder(self.manager, DEV, 1 << 30, self.status)

    def step(self, portions: Dict[str, int]):
        """portions: request -> number of new tokens.  Returns the StepContext."""
        from atom_b200.engine.batch import StepEntry

        entries, targets = [], []
        for rid, n in portions.items():
            if rid not in self.manager.requests:
                self.manager.admit(rid)
            t = self.manager.committed(rid) + n
            self.manager.extend(rid, t)
            entries.append(StepEntry(rid, [0] * n, ()))
            targets.append(t)
        ctx = self.builder.build(entries, targets)
        self._pending = list(zip(portions, targets))
        return ctx

    def commit(self):
        for rid, t in self._pending:
            self.manager.commit(rid, t)


# ----------------------------------------------------------------------------- norm, position, embedding, head


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, T, eps = 200, 6, 3e-6
    rt = _rt(dtype)
    norm = registry.build("norm", PartSpec("rmsnorm", {"size": H, "eps": eps}))
    w = _bind(norm, {"weight": _rand((H,), 1, 0.1) + 1}, rt)["weight"]
    res = _rand((T, H), 2).float().to(DEV)
    delta = _rand((T, H), 3).to(dtype).to(DEV)
    want_res = res.double().cpu() + delta.double().cpu()
    out = norm.add_norm(res, delta, "t")
    torch.testing.assert_close(res.double().cpu(), want_res, rtol=1e-6, atol=1e-6)
    want = plain.rms_norm(want_res, w, eps)
    torch.testing.assert_close(out.double().cpu(), want, **_tol(dtype))


def test_rotary_table_part():
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    rd, theta, n = 48, 500000.0, 300
    pos = registry.build("position", PartSpec("rope_neox", {"rotary_dim": rd, "theta": theta, "max_position": n}))
    table = pos.table(_rt(torch.float32)).cpu()
    cos, sin = plain.rope_cos_sin(torch.arange(n), rd, theta)
    assert table.shape == (n, rd)
    torch.testing.assert_close(table[:, : rd // 2], cos, rtol=0, atol=2e-6)
    torch.testing.assert_close(table[:, rd // 2:], sin, rtol=0, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head_parts(dtype, tied):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    V, H = 301, 192
    rt = _rt(dtype)
    emb = registry.build("embedding", PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}))
    head = registry.build("head", PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": tied}))
    E = _bind(emb, {"weight": _rand((V, H), 4, 0.05)}, rt)["weight"]
    if tied:
        head.bind({}, rt)
        head.tie(emb)
        W = E
    else:
        W = _bind(head, {"weight": _rand((V, H), 5, 0.05)}, rt)["weight"]
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    r = emb.forward(ids, 5)
    assert r.dtype == torch.float32
    torch.testing.assert_close(r.double().cpu(), E[ids.long().cpu()], rtol=0, atol=0)
    x = _rand((3, H), 6).to(dtype).to(DEV)
    logits = head.forward(x)
    assert logits.dtype == torch.float32 and logits.shape == (3, V)
    torch.testing.assert_close(logits.double().cpu(), x.double().cpu() @ W.T, **_tol(dtype))


# ----------------------------------------------------------------------------- feed-forward, mixer, block


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 40])          # few rows: fused kernel; many rows: library product + activation
def test_gated_silu_part(dtype, T):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, I = 192, 320
    rt = _rt(dtype)
    ffn = registry.build("ffn", PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": I}))
    w = _bind(ffn, {"gate_up.weight": _rand((2 * I, H), 7, 0.08), "down.weight": _rand((H, I), 8, 0.08)}, rt)
    x = _rand((T, H), 9).to(dtype).to(DEV)
    got = ffn.forward(x, None)
    xd = x.double().cpu()
    want = plain.silu_and_mul(xd @ w["gate_up.weight"].T) @ w["down.weight"].T
    torch.testing.assert_close(got.double().cpu(), want, **_tol(dtype))


def _attention_part(dtype, window=None, bias=False):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, nh, nkv, hd, eps, theta = 160, 6, 3, 32, 1e-5, 10000.0
    rt = _rt(dtype)
    spec = PartSpec("paged_attention", dict(
        hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, qk_norm=True, norm_eps=eps, bias=bias,
        window=window, position=PartSpec("rope_neox", {"rotary_dim": hd, "theta": theta, "max_position": 512})))
    attn = registry.build("mixer", spec)
    q, kv = nh * hd, nkv * hd
    t = {"qkv.weight": _rand((q + 2 * kv, H), 10, 0.08), "o.weight": _rand((H, q), 11, 0.08),
         "q_norm.weight": (_rand((hd,), 12, 0.1) + 1) * 2, "k_norm.weight": (_rand((hd,), 13, 0.1) + 1) * 2}
    if bias:
        t["qkv.bias"] = _rand((q + 2 * kv,), 14, 0.05)
    w = _bind(attn, t, rt)
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, hidden_size=H, rms_norm_eps=eps,
               rope_theta=theta, attention_bias=bias)
    pw = {"a.q_proj.weight": w["qkv.weight"][:q], "a.k_proj.weight": w["qkv.weight"][q:q + kv],
          "a.v_proj.weight": w["qkv.weight"][q + kv:], "a.o_proj.weight": w["o.weight"],
          "a.q_norm.weight": w["q_norm.weight"], "a.k_norm.weight": w["k_norm.weight"]}
    if bias:
        pw.update({"a.q_proj.bias": w["qkv.bias"][:q], "a.k_proj.bias": w["qkv.bias"][q:q + kv],
                   "a.v_proj.bias": w["qkv.bias"][q + kv:]})
    return attn, cfg, pw, H


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,bias", [(None, False), (20, True)])
def test_attention_part_whole_and_in_portions(dtype, window, bias):
    attn, cfg, pw, H = _attention_part(dtype, window, bias)
    lens = {"a": 70, "b": 33}
    x = {r: _rand((n, H), 20 + i).to(dtype) for i, (r, n) in enumerate(lens.items())}
    want = {r: plain.attention_block(x[r].double(), pw, "a", cfg, torch.arange(n), window)
            for r, n in lens.items()}
    # whole, both requests in one batch
    c = _Cache(attn.cache_need(), dtype)
    ctx = c.step(lens)
    got = attn.forward(torch.cat([x["a"], x["b"]]).to(DEV), ctx, c.storage.view(0), True).double().cpu()
    c.commit()
    _assert_mixer_close(got[:70], want["a"], dtype)
    _assert_mixer_close(got[70:], want["b"], dtype)
    assert int(c.status.item()) == 0
    # in portions: a in 37 + 2 + 31, b whole beside a's second portion, then a decodes its last token
    c = _Cache(attn.cache_need(), dtype)
    outs = {"a": [], "b": []}
    done = {"a": 0, "b": 0}
    for portions in ({"a": 37}, {"a": 2, "b": 33}, {"a": 30}, {"a": 1}):
        ctx = c.step(portions)
        xs = torch.cat([x[r][done[r]:done[r] + n] for r, n in portions.items()]).to(DEV)
        y = attn.forward(xs, ctx, c.storage.view(0), True).double().cpu()
        c.commit()
        o = 0
        for r, n in portions.items():
            outs[r].append(y[o:o + n])
            done[r] += n
            o += n
    for r in lens:
        _assert_mixer_close(torch.cat(outs[r]), want[r], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block(dtype):
    """norm -> mixer -> norm -> feed-forward around the 32-bit residual (one block, then the
    closing add that the next norm would do)."""
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    attn, cfg, pw, H = _attention_part(dtype)
    rt = attn.rt
    I, eps = 224, 1e-5
    n1 = registry.build("norm", PartSpec("rmsnorm", {"size": H, "eps": eps}))
    n2 = registry.build("norm", PartSpec("rmsnorm", {"size": H, "eps": eps}))
    ffn = registry.build("ffn", PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": I}))
    w1 = _bind(n1, {"weight": _rand((H,), 30, 0.1) + 1}, rt)["weight"]
    w2 = _bind(n2, {"weight": _rand((H,), 31, 0.1) + 1}, rt)["weight"]
    wf = _bind(ffn, {"gate_up.weight": _rand((2 * I, H), 32, 0.08), "down.weight": _rand((H, I), 33, 0.08)}, rt)
    block = registry.lookup("arrangement", "prenorm")(n1, attn, n2, ffn)
    T = 29
    r0 = _rand((T, H), 34).float()
    res = r0.clone().to(DEV)
    c = _Cache(attn.cache_need(), dtype)
    ctx = c.step({"a": T})
    delta = block.run(res, None, ctx, c.storage.view(0), True)
    got = res.double().cpu() + delta.double().cpu()
    r = r0.double()
    r = r + plain.attention_block(plain.rms_norm(r, w1, eps), pw, "a", cfg, torch.arange(T), None)
    b = plain.rms_norm(r, w2, eps)
    r = r + plain.silu_and_mul(b @ wf["gate_up.weight"].T) @ wf["down.weight"].T
    _assert_mixer_close(got, r, dtype)


# ----------------------------------------------------------------------------- a toy mixer with state


def _register_toy():
    """A mixer that keeps a running, decayed sum of its projected inputs per request:
         s_t = d * s_(t-1) + W x_t,   y_t = s_t      (s = 0 before the request's first token)
    Its state is one float32 vector per request, held in the request's state slot.  It is a
    toy for this test: plain torch on the device, nothing of it is in the framework."""
    from atom_b200.config.model_config import ModelConfig
    from atom_b200.models.registry import register_architecture
    from atom_b200.parts import registry
    from atom_b200.parts.base import Mixer
    from atom_b200.parts.spec import CacheNeed, LayerSpec, ModelSpec, ParamSpec, PartSpec, RunEntry

    if "toy_decay_sum" in registry._REGISTRIES["mixer"]:
        return

    @registry.register("mixer", "toy_decay_sum")
    class DecaySum(Mixer):
        def __init__(self, hidden_size: int):
            self.hidden_size = hidden_size

        def params(self):
            H = self.hidden_size
            return {"in.weight": ParamSpec((H, H)), "decay": ParamSpec((H,), role="vector", init="norm")}

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.hidden_size,), state_dtype="float32")

        def forward(self, x, step, cache, writes_cache):
            u = (x.float() @ self.w_in_weight.float().T)
            d = self.w_decay.float() * 0.5
            y = torch.empty_like(u)
            t = 0
            for i, n in enumerate(step.q_lens):
                slot = step.host_state_slots[i]
                s = cache.state[slot]
                if step.q_starts[i] == 0:
                    s.zero_()
                for k in range(n):
                    s.mul_(d).add_(u[t + k])
                    y[t + k] = s
                t += n
            return y.to(self.rt.dtype)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 0
        num_hidden_layers: int = 0
        vocab_size: int = 0
        intermediate_size: int = 0
        eps: float = 1e-5

        def to_dict(self) -> Dict[str, Any]:
            return {"architectures": [self.architecture], "hidden_size": self.hidden_size,
                    "num_hidden_layers": self.num_hidden_layers, "vocab_size": self.vocab_size,
                    "intermediate_size": self.intermediate_size, "eps": self.eps}

    def from_dict(d):
        return ToyConfig("ToyRecurrentLM", d["hidden_size"], d["num_hidden_layers"], d["vocab_size"],
                         d["intermediate_size"], d["eps"])

    def build_spec(cfg):
        H = cfg.hidden_size
        pos = PartSpec("rope_neox", {"rotary_dim": 16, "theta": 10000.0, "max_position": 512})
        layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"l{i}"
            if i % 2 == 0:
                mixer = PartSpec("toy_decay_sum", {"hidden_size": H},
                                 {"in.weight": (f"{p}.mix.in",), "decay": (f"{p}.mix.decay",)})
            else:
                mixer = PartSpec("paged_attention",
                                 dict(hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16, position=pos,
                                      qk_norm=False),
                                 {"qkv.weight": (f"{p}.q", f"{p}.k", f"{p}.v"), "o.weight": (f"{p}.o",)})
            norm = lambda n: PartSpec("rmsnorm", {"size": H, "eps": cfg.eps}, {"weight": (f"{p}.{n}",)})
            ffn = PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": cfg.intermediate_size},
                           {"gate_up.weight": (f"{p}.gate", f"{p}.up"), "down.weight": (f"{p}.down",)})
            layers.append(LayerSpec("prenorm", dict(mixer_norm=norm("n1"), mixer=mixer, ffn_norm=norm("n2"), ffn=ffn)))
        return ModelSpec(
            architecture=cfg.architecture, hidden_size=H, vocab_size=cfg.vocab_size, max_position=512,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H}, {"weight": ("emb",)}),
            layers=tuple(layers), run_order=tuple(RunEntry(i, i) for i in range(cfg.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.eps}, {"weight": ("norm",)}),
            lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "tied": True}, {}))

    register_architecture("ToyRecurrentLM", from_dict, build_spec)


def _toy_plain(model_dir, tokens):
    """The toy architecture written out plainly: whole sequence, float64, no cache."""
    cfg = plain.read_config(model_dir)
    w = plain.read_tensors(model_dir)
    H, eps = cfg["hidden_size"], cfg["eps"]
    T = len(tokens)
    r = w["emb"][torch.as_tensor(tokens)]
    att_cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16, hidden_size=H, rms_norm_eps=eps,
                   rope_theta=10000.0)
    for i in range(cfg["num_hidden_layers"]):
        p = f"l{i}"
        a = plain.rms_norm(r, w[f"{p}.n1"], eps)
        if i % 2 == 0:
            u = a @ w[f"{p}.mix.in"].T
            d = w[f"{p}.mix.decay"] * 0.5
            s = torch.zeros(H, dtype=torch.float64)
            m = torch.empty_like(u)
            for t in range(T):
                s = d * s + u[t]
                m[t] = s
        else:
            q = (a @ w[f"{p}.q"].T).view(T, 4, 16)
            k = (a @ w[f"{p}.k"].T).view(T, 2, 16)
            v = (a @ w[f"{p}.v"].T).view(T, 2, 16)
            cos, sin = plain.rope_cos_sin(torch.arange(T), 16, 10000.0)
            o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, 16 ** -0.5)
            m = o.reshape(T, 64) @ w[f"{p}.o"].T
        r = r + m
        b = plain.rms_norm(r, w[f"{p}.n2"], eps)
        gu = torch.cat((b @ w[f"{p}.gate"].T, b @ w[f"{p}.up"].T), dim=-1)
        r = r + plain.silu_and_mul(gu) @ w[f"{p}.down"].T
    return (plain.rms_norm(r, w["norm"], eps) @ w["emb"].T).numpy()


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from atom_b200.config import EngineConfig, config_from_dict
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner
    from atom_b200.weights import write_random_model

    _register_toy()
    cfg = config_from_dict({"architectures": ["ToyRecurrentLM"], "hidden_size": 64, "num_hidden_layers": 4,
                            "vocab_size": 97, "intermediate_size": 80, "eps": 1e-5})
    d = str(tmp_path / "toy")
    write_random_model(d, cfg, seed=21)
    runner = ModelRunner(EngineConfig(model=d, dtype="float32", kv_cache_block_size=8, num_kvcache_blocks=32,
                                      max_num_seqs=4, enforce_eager=True))
    assert len(runner.cache.state_needs) == 2 and len(runner.cache.groups) == 1
    rng = np.random.default_rng(3)
    seqs = {"x": rng.integers(0, 97, 41).tolist(), "y": rng.integers(0, 97, 23).tolist(),
            "z": rng.integers(0, 97, 9).tolist()}
    ref = {r: _toy_plain(d, t) for r, t in seqs.items()}
    got = {r: [] for r in seqs}
    done = {r: 0 for r in seqs}
    # portions of some beside single tokens of others; z enters after y has ended and takes its slot
    plan = [{"x": 17}, {"x": 2, "y": 20}, {"x": 1, "y": 1}, {"x": 20, "y": 2}, {"x": 1, "z": 9}]
    for portions in plan:
        entries = [StepEntry(r, seqs[r][done[r]:done[r] + n], list(range(n))) for r, n in portions.items()]
        logits = runner.step(entries).cpu().numpy()
        o = 0
        for r, n in portions.items():
            got[r].append(logits[o:o + n])
            o += n
            done[r] += n
            if done[r] == len(seqs[r]):
                runner.finish(r)
    runner.check_status()
    for r in seqs:
        assert done[r] == len(seqs[r])
        err = np.abs(np.concatenate(got[r]) - ref[r]).max()
        assert err < 2e-4, f"{r}: max abs error {err:.2e}"
    assert runner.cache.state_slots.num_free == 4


# ----------------------------------------------------------------------------- layers with different mixers


def _register_hybrid():
    from dataclasses import dataclass
    from typing import Any, Dict

    from atom_b200.config.model_config import ModelConfig
    from atom_b200.models.registry import register_architecture, registered_architectures
    from atom_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

    if "ToyHybridLM" in registered_architectures():
        return

    @dataclass(frozen=True)
    class HybridConfig(ModelConfig):
        hidden_size: int = 0
        vocab_size: int = 0
        window: int = 0

        def to_dict(self) -> Dict[str, Any]:
            return {"architectures": [self.architecture], "hidden_size": self.hidden_size,
                    "vocab_size": self.vocab_size, "window": self.window}

    def from_dict(d):
        return HybridConfig("ToyHybridLM", d["hidden_size"], d["vocab_size"], d["window"])

    def build_spec(cfg):
        H = cfg.hidden_size
        pos = PartSpec("rope_neox", {"rotary_dim": 128, "theta": 10000.0, "max_position": 1024})
        layers = []
        for i, window in enumerate((None, cfg.window, None)):   # all keys, a window, all keys: same head counts
            p = f"l{i}"
            mixer = PartSpec("paged_attention",
                             dict(hidden_size=H, num_heads=2, num_kv_heads=1, head_dim=128, position=pos, qk_norm=False,
                                  window=window),
                             {"qkv.weight": (f"{p}.q", f"{p}.k", f"{p}.v"), "o.weight": (f"{p}.o",)})
            norm = lambda n: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, {"weight": (f"{p}.{n}",)})
            ffn = PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": 2 * H},
                           {"gate_up.weight": (f"{p}.gate", f"{p}.up"), "down.weight": (f"{p}.down",)})
            layers.append(LayerSpec("prenorm", dict(mixer_norm=norm("n1"), mixer=mixer, ffn_norm=norm("n2"), ffn=ffn)))
        return ModelSpec(
            architecture=cfg.architecture, hidden_size=H, vocab_size=cfg.vocab_size, max_position=1024,
            embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H}, {"weight": ("emb",)}),
            layers=tuple(layers), run_order=tuple(RunEntry(i, i) for i in range(3)),
            final_norm=PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, {"weight": ("norm",)}),
            lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "tied": True}, {}))

    register_architecture("ToyHybridLM", from_dict, build_spec)


def _hybrid_plain(model_dir, tokens, window):
    w = plain.read_tensors(model_dir)
    T = len(tokens)
    r = w["emb"][torch.as_tensor(tokens)]
    cos, sin = plain.rope_cos_sin(torch.arange(T), 128, 10000.0)
    for i, win in enumerate((None, window, None)):
        p = f"l{i}"
        a = plain.rms_norm(r, w[f"{p}.n1"], 1e-5)
        q = (a @ w[f"{p}.q"].T).view(T, 2, 128)
        k = (a @ w[f"{p}.k"].T).view(T, 1, 128)
        v = (a @ w[f"{p}.v"].T).view(T, 1, 128)
        o = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, 128 ** -0.5, win)
        r = r + o.reshape(T, 256) @ w[f"{p}.o"].T
        b = plain.rms_norm(r, w[f"{p}.n2"], 1e-5)
        r = r + plain.silu_and_mul(torch.cat((b @ w[f"{p}.gate"].T, b @ w[f"{p}.up"].T), dim=-1)) @ w[f"{p}.down"].T
    return (plain.rms_norm(r, w["norm"], 1e-5) @ w["emb"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_beside_layers_without(tmp_path, dtype):
    """Layers of one model choose their mixers' options one by one: all keys in layers 0 and 2, a window in
    layer 1, with the same head counts.  The long portion runs on the tcgen05 kernel in layers 0 and 2 only
    (a launch plan made for them must not be handed to layer 1); the windowed layer's pages are given back
    as the window passes them (two page groups)."""
    from atom_b200.config import EngineConfig, config_from_dict
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner
    from atom_b200.weights import write_random_model

    _register_hybrid()
    window = 48
    cfg = config_from_dict({"architectures": ["ToyHybridLM"], "hidden_size": 96, "vocab_size": 211, "window": window})
    d = str(tmp_path / "hybrid")
    write_random_model(d, cfg, seed=5)
    runner = ModelRunner(EngineConfig(model=d, dtype=dtype, kv_cache_block_size=16, num_kvcache_blocks=40,
                                      max_num_seqs=4, enforce_eager=True))
    assert len(runner.cache.groups) == 2
    rng = np.random.default_rng(9)
    toks = rng.integers(0, 211, 230).tolist()
    ref = _hybrid_plain(d, toks, window)
    got, done = [], 0
    for n in (150, 1, 70, 2, 7):            # 300 packed rows at once, then single tokens and portions
        got.append(runner.step([StepEntry("a", toks[done:done + n], list(range(n)))]).cpu().numpy())
        done += n
    runner.check_status()
    got = np.concatenate(got)
    err = np.abs(got - ref).max()
    scale = np.abs(ref).max()
    assert err < (2e-4 if dtype == "float32" else 0.08 * scale), f"max abs error {err:.2e} (scale {scale:.2f})"
    used = [g.pool.num_used for g in runner.cache.groups]
    assert min(used) < max(used)            # the windowed group holds fewer pages than the full one
    runner.finish("a")
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


# ----------------------------------------------------------------------------- a toy feed-forward with routing, another position encoding


def _register_routed():
    """Two toys for this test, plain torch on the device, nothing of them in the framework:

    * a feed-forward with routing: router logits in 32-bit, the ``top_k`` largest of ``num_experts``, their
      softmax as weights, each chosen expert a SiLU-gated feed-forward of its own:
          y = sum_{e in top_k(x W_r^T)} softmax_e * down_e(silu(gate_e x) * up_e x)
    * another position encoding: rotation of the first ``rotary_dim`` < head size entries of a head only, by
      angles  (pos / stretch + shift) * theta^(-2j/rotary_dim): a stretched and shifted table.
    The model runs the routed feed-forward in the odd layers and the dense one in the even layers."""
    from dataclasses import dataclass
    from typing import Any, Dict

    from atom_b200.config.model_config import ModelConfig
    from atom_b200.models.registry import register_architecture, registered_architectures
    from atom_b200.parts import registry
    from atom_b200.parts.base import FeedForward, PositionEncoding
    from atom_b200.parts.spec import LayerSpec, ModelSpec, ParamSpec, PartSpec, RunEntry

    if "ToyRoutedLM" in registered_architectures():
        return

    @registry.register("ffn", "toy_routed_silu")
    class RoutedSilu(FeedForward):
        def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int):
            self.H, self.I, self.E, self.k = hidden_size, intermediate_size, num_experts, top_k

        def params(self):
            return {"router.weight": ParamSpec((self.E, self.H)),
                    "gate_up.weight": ParamSpec((self.E * 2 * self.I, self.H), rows=(2 * self.I,) * self.E),
                    "down.weight": ParamSpec((self.E * self.H, self.I), rows=(self.H,) * self.E)}

        def forward(self, x, step):
            xf = x.float()
            logits = xf @ self.w_router_weight.float().T
            top, idx = logits.topk(self.k, dim=-1)
            wts = torch.softmax(top, dim=-1)
            gu = self.w_gate_up_weight.float().view(self.E, 2 * self.I, self.H)
            dn = self.w_down_weight.float().view(self.E, self.H, self.I)
            y = torch.zeros_like(xf)
            for e in range(self.E):
                rows, slot = (idx == e).nonzero(as_tuple=True)
                if rows.numel():
                    h = xf[rows] @ gu[e].T
                    h = torch.nn.functional.silu(h[:, :self.I]) * h[:, self.I:]
                    y.index_add_(0, rows, (h @ dn[e].T) * wts[rows, slot].unsqueeze(1))
            return y.to(self.rt.dtype)

    @registry.register("position", "toy_stretched_rotary")
    class StretchedRotary(PositionEncoding):
        def __init__(self, rotary_dim: int, theta: float, max_position: int, stretch: float, shift: float):
            self.rotary_dim, self.theta, self.max_position = rotary_dim, theta, max_position
            self.stretch, self.shift = stretch, shift

        def table(self, rt):
            d = self.rotary_dim
            inv = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
            ang = torch.outer(torch.arange(self.max_position, dtype=torch.float64) / self.stretch + self.shift, inv)
            return torch.cat([ang.cos(), ang.sin()], dim=1).float().contiguous().to(rt.device)

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        d: Any = None

        def to_dict(self) -> Dict[str, Any]:
            return dict(self.d)

    def from_dict(d):
        return RoutedConfig("ToyRoutedLM", dict(d))

    def build_spec(cfg):
        c = cfg.d
        H, hd, nh, nkv = c["hidden_size"], c["head_dim"], c["heads"], c["kv_heads"]
        pos = PartSpec("toy_stretched_rotary", {"rotary_dim": c["rotary_dim"], "theta": c["theta"], "max_position": 256,
                                                "stretch": c["stretch"], "shift": c["shift"]})
        layers = []
        for i in range(c["layers"]):
            p = f"l{i}"
            mixer = PartSpec("paged_attention",
                             dict(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, position=pos, qk_norm=True,
                                  norm_eps=c["eps"]),
                             {"qkv.weight": (f"{p}.q", f"{p}.k", f"{p}.v"), "o.weight": (f"{p}.o",),
                              "q_norm.weight": (f"{p}.qn",), "k_norm.weight": (f"{p}.kn",)})
            if i % 2:
                E = c["experts"]
                ffn = PartSpec("toy_routed_silu", {"hidden_size": H, "intermediate_size": c["expert_size"],
                                                   "num_experts": E, "top_k": c["top_k"]},
                               {"router.weight": (f"{p}.router",),
                                "gate_up.weight": tuple(f"{p}.e{e}.gate_up" for e in range(E)),
                                "down.weight": tuple(f"{p}.e{e}.down" for e in range(E))})
            else:
                ffn = PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": c["dense_size"]},
                               {"gate_up.weight": (f"{p}.gate", f"{p}.up"), "down.weight": (f"{p}.down",)})
            norm = lambda n: PartSpec("rmsnorm", {"size": H, "eps": c["eps"]}, {"weight": (f"{p}.{n}",)})
            layers.append(LayerSpec("prenorm", dict(mixer_norm=norm("n1"), mixer=mixer, ffn_norm=norm("n2"), ffn=ffn)))
        return ModelSpec(
            architecture=cfg.architecture, hidden_size=H, vocab_size=c["vocab_size"], max_position=256,
            embedding=PartSpec("token_embedding", {"vocab_size": c["vocab_size"], "hidden_size": H}, {"weight": ("emb",)}),
            layers=tuple(layers), run_order=tuple(RunEntry(i, i) for i in range(c["layers"])),
            final_norm=PartSpec("rmsnorm", {"size": H, "eps": c["eps"]}, {"weight": ("norm",)}),
            lm_head=PartSpec("lm_head", {"vocab_size": c["vocab_size"], "hidden_size": H, "tied": False},
                             {"weight": ("head",)}))

    register_architecture("ToyRoutedLM", from_dict, build_spec)


def _routed_plain(model_dir, tokens):
    """The toy architecture written out plainly: whole sequence, float64, no cache."""
    c = plain.read_config(model_dir)
    w = plain.read_tensors(model_dir)
    H, hd, nh, nkv, eps, rd = c["hidden_size"], c["head_dim"], c["heads"], c["kv_heads"], c["eps"], c["rotary_dim"]
    T = len(tokens)
    inv = 1.0 / (c["theta"] ** (torch.arange(0, rd, 2, dtype=torch.float64) / rd))
    ang = torch.outer(torch.arange(T, dtype=torch.float64) / c["stretch"] + c["shift"], inv)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rotate(x):                       # the first rd entries of every head, half-split pairs; the rest untouched
        x1, x2, rest = x[..., :rd // 2], x[..., rd // 2:rd], x[..., rd:]
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest), dim=-1)

    r = w["emb"][torch.as_tensor(tokens)]
    for i in range(c["layers"]):
        p = f"l{i}"
        a = plain.rms_norm(r, w[f"{p}.n1"], eps)
        q = plain.rms_norm((a @ w[f"{p}.q"].T).view(T, nh, hd), w[f"{p}.qn"], eps)
        k = plain.rms_norm((a @ w[f"{p}.k"].T).view(T, nkv, hd), w[f"{p}.kn"], eps)
        v = (a @ w[f"{p}.v"].T).view(T, nkv, hd)
        o = plain.causal_attention(rotate(q), rotate(k), v, hd ** -0.5)
        r = r + o.reshape(T, nh * hd) @ w[f"{p}.o"].T
        b = plain.rms_norm(r, w[f"{p}.n2"], eps)
        if i % 2:
            logits = b @ w[f"{p}.router"].T
            y = torch.zeros_like(b)
            for t in range(T):
                top = torch.topk(logits[t], c["top_k"])
                wt = torch.softmax(top.values, dim=-1)
                for j, e in enumerate(top.indices.tolist()):
                    y[t] += wt[j] * (plain.silu_and_mul(b[t:t + 1] @ w[f"{p}.e{e}.gate_up"].T) @ w[f"{p}.e{e}.down"].T)[0]
            r = r + y
        else:
            r = r + plain.silu_and_mul(torch.cat((b @ w[f"{p}.gate"].T, b @ w[f"{p}.up"].T), dim=-1)) @ w[f"{p}.down"].T
    return (plain.rms_norm(r, w["norm"], eps) @ w["head"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    """A feed-forward with routing and a position encoding of another kind, both defined here, are registered, chosen
    layer by layer beside the framework's dense feed-forward, loaded by tensor name (an expert's matrices are
    checkpoint tensors of their own) and stepped in portions beside decoded tokens, without a change to the framework."""
    from atom_b200.config import EngineConfig, config_from_dict
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner
    from atom_b200.weights import write_random_model

    _register_routed()
    cfg = config_from_dict({"architectures": ["ToyRoutedLM"], "hidden_size": 80, "head_dim": 32, "heads": 6, "kv_heads": 3,
                            "layers": 4, "vocab_size": 131, "eps": 1e-5, "rotary_dim": 16, "theta": 500.0, "stretch": 2.5,
                            "shift": 0.75, "experts": 5, "top_k": 2, "expert_size": 48, "dense_size": 112})
    d = str(tmp_path / "routed")
    write_random_model(d, cfg, seed=33)
    # router rows drawn like every matrix would leave the choice of experts to differences of 1e-3: scale them up
    # so that the plain implementation and the engine choose alike also in reduced precision
    from safetensors.torch import load_file, save_file
    t = load_file(os.path.join(d, "model.safetensors"))
    for k_ in t:
        if k_.endswith(".router"):
            t[k_] = (t[k_].float() * 40).to(t[k_].dtype)
    save_file(t, os.path.join(d, "model.safetensors"))
    runner = ModelRunner(EngineConfig(model=d, dtype=dtype, kv_cache_block_size=8, num_kvcache_blocks=32,
                                      max_num_seqs=4, enforce_eager=True))
    rng = np.random.default_rng(4)
    seqs = {"x": rng.integers(0, 131, 50).tolist(), "y": rng.integers(0, 131, 21).tolist()}
    ref = {r: _routed_plain(d, s) for r, s in seqs.items()}
    got, done = {r: [] for r in seqs}, {r: 0 for r in seqs}
    for portions in ({"x": 19}, {"x": 2, "y": 20}, {"x": 1, "y": 1}, {"x": 27}, {"x": 1}):
        entries = [StepEntry(r, seqs[r][done[r]:done[r] + n], list(range(n))) for r, n in portions.items()]
        logits = runner.step(entries).cpu().numpy()
        o = 0
        for r, n in portions.items():
            got[r].append(logits[o:o + n])
            o += n
            done[r] += n
    runner.check_status()
    for r in seqs:
        assert done[r] == len(seqs[r])
        err = np.abs(np.concatenate(got[r]) - ref[r])
        if dtype == "float32":
            assert err.max() < 2e-4, f"{r}: max abs error {err.max():.2e}"
        else:
            # a token whose second and third router logits are closer than bfloat16 resolves may take another
            # expert: all but a few rows must agree closely
            scale = np.abs(ref[r]).max()
            bad = (err.max(axis=1) > 0.08 * scale).sum()
            assert bad <= 2, f"{r}: {bad} rows off (max abs error {err.max():.2e}, scale {scale:.2f})"


# ----------------------------------------------------------------------------- four norms, one cached row per token, positions on a grid


def _register_sandwich():
    """Three things a layer of the built-in kind does not have, each defined here and none of it in the
    framework (toys for this test; plain torch on the device):

    * an arrangement with four norms, "toy_sandwich": a norm before and a norm after the mixer and the same
      around the feed-forward, the second of each applied to the sub-block's output before it joins the
      residual stream; the feed-forward and its norms may be absent from a layer:
          r += delta;  m = post_mixer(mixer(pre_mixer(r)));  r += m;  delta' = post_ffn(ffn(pre_ffn(r)))
    * a mixer that keeps ONE row of ``rank`` numbers per token in pages (not keys and values per head):
          c_t = W_c x_t;  q_t = W_q x_t;  p = softmax_{j <= t}(q_t . c_j / sqrt(rank));  y_t = W_o sum_j p_j c_j
      with a side-by-side parameter ``qc.weight`` = [W_q | W_c]^T stacked along dim 1 of the checkpoint;
    * a position encoding that is no table of angles by position: tokens lie on a grid ``width`` wide, the
      first half of a head is rotated by the row's angle and the second half by the column's.
    """
    from atom_b200.config.model_config import ModelConfig
    from atom_b200.models.registry import register_architecture, registered_architectures
    from atom_b200.parts import registry
    from atom_b200.parts.base import Mixer, PositionEncoding
    from atom_b200.parts.spec import CacheEntry, CacheNeed, LayerSpec, ModelSpec, ParamSpec, PartSpec, RunEntry

    if "ToySandwichLM" in registered_architectures():
        return

    @registry.register("arrangement", "toy_sandwich")
    class Sandwich:
        slots = {"pre_mixer": "norm", "mixer": "mixer", "post_mixer": "norm",
                 "pre_ffn": "norm", "ffn": "ffn", "post_ffn": "norm"}
        optional = ("pre_ffn", "ffn", "post_ffn")

        def __init__(self, pre_mixer, mixer, post_mixer, pre_ffn=None, ffn=None, post_ffn=None):
            self.pre_mixer, self.mixer, self.post_mixer = pre_mixer, mixer, post_mixer
            self.pre_ffn, self.ffn, self.post_ffn = pre_ffn, ffn, post_ffn

        def run(self, residual, delta, step, cache, writes_cache):
            a = self.pre_mixer.add_norm(residual, delta, "sw.pre_mixer")
            m = self.mixer.forward(a, step, cache, writes_cache)
            m = self.post_mixer.add_norm(m.float(), None, "sw.post_mixer")
            if self.ffn is None:
                return m
            b = self.pre_ffn.add_norm(residual, m, "sw.pre_ffn")
            f = self.ffn.forward(b, step)
            return self.post_ffn.add_norm(f.float(), None, "sw.post_ffn")

    @registry.register("mixer", "toy_latent_rows")
    class LatentRows(Mixer):
        def __init__(self, hidden_size: int, rank: int):
            self.H, self.r = hidden_size, rank

        def params(self):
            return {"qc.weight": ParamSpec((self.H, 2 * self.r), rows=(self.r, self.r), stack_dim=1),
                    "o.weight": ParamSpec((self.H, self.r))}

        def cache_need(self):
            return CacheNeed("pages", entries=(CacheEntry("latent", (self.r,), "float32"),))

        def forward(self, x, step, cache, writes_cache):
            qc = x.float() @ self.w_qc_weight.float()
            q, c = qc[:, :self.r], qc[:, self.r:]
            pages = cache.pages["latent"]                 # [pages, page size, rank]
            assert pages.shape[1:] == (cache.page_size, self.r) and pages.dtype == torch.float32
            table = step.block_tables[cache.group]
            y = torch.empty_like(q)
            t = 0
            for i, n in enumerate(step.q_lens):
                start = step.q_starts[i]
                pos = torch.arange(start + n, device=x.device)
                where = table[i, pos // cache.page_size].long() * cache.page_size + pos % cache.page_size
                flat = pages.view(-1, self.r)
                if writes_cache:
                    flat[where[start:]] = c[t:t + n]
                rows = flat[where]                          # the request's rows, old and new
                s = (q[t:t + n] @ rows.T) * self.r ** -0.5
                s = s.masked_fill(pos[None, :] > pos[start:, None], float("-inf"))
                y[t:t + n] = torch.softmax(s, dim=-1) @ rows
                t += n
            return (y @ self.w_o_weight.float().T).to(self.rt.dtype)

    @registry.register("position", "toy_grid_rotary")
    class GridRotary(PositionEncoding):
        def __init__(self, head_dim: int, width: int, theta: float):
            self.hd, self.width, self.theta = head_dim, width, theta

        def apply(self, q, k, step):
            pos = step.positions.long()
            half = self.hd // 2
            inv = 1.0 / (self.theta ** (torch.arange(0, half, 2, dtype=torch.float32, device=q.device) / half))
            for x in (q, k):
                for part, p in ((x[..., :half], pos // self.width), (x[..., half:], pos % self.width)):
                    ang = p.float()[:, None] * inv[None, :]
                    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
                    a, b = part[..., :half // 2].float().clone(), part[..., half // 2:].float().clone()
                    part[..., :half // 2] = (a * cos - b * sin).to(x.dtype)
                    part[..., half // 2:] = (b * cos + a * sin).to(x.dtype)

    @dataclass(frozen=True)
    class SandwichConfig(ModelConfig):
        d: Any = None

        def to_dict(self) -> Dict[str, Any]:
            return dict(self.d)

    def from_dict(d):
        return SandwichConfig("ToySandwichLM", tuple(sorted(d.items())))

    def build_spec(cfg):
        c = dict(cfg.d)
        H = c["hidden_size"]
        grid = PartSpec("toy_grid_rotary", {"head_dim": c["head_dim"], "width": c["grid_width"], "theta": 100.0})
        layers = []
        for i in range(c["num_hidden_layers"]):
            p = f"l{i}"
            norm = lambda n: PartSpec("rmsnorm", {"size": H, "eps": c["eps"]}, {"weight": (f"{p}.{n}",)})
            if i % 2 == 0:
                mixer = PartSpec("toy_latent_rows", {"hidden_size": H, "rank": c["rank"]},
                                 {"qc.weight": (f"{p}.wq", f"{p}.wc"), "o.weight": (f"{p}.wo",)})
            else:
                mixer = PartSpec("paged_attention",
                                 dict(hidden_size=H, num_heads=c["heads"], num_kv_heads=1, head_dim=c["head_dim"],
                                      position=grid, qk_norm=True, norm_eps=c["eps"]),
                                 {"qkv.weight": (f"{p}.q", f"{p}.k", f"{p}.v"), "o.weight": (f"{p}.o",),
                                  "q_norm.weight": (f"{p}.qn",), "k_norm.weight": (f"{p}.kn",)})
            parts = {"pre_mixer": norm("n1"), "mixer": mixer, "post_mixer": norm("n2")}
            if i != 1:                                # layer 1 has no feed-forward at all
                parts.update({"pre_ffn": norm("n3"), "post_ffn": norm("n4"),
                              "ffn": PartSpec("gated_silu", {"hidden_size": H, "intermediate_size": c["inter"]},
                                              {"gate_up.weight": (f"{p}.gate", f"{p}.up"),
                                               "down.weight": (f"{p}.down",)})})
            layers.append(LayerSpec("toy_sandwich", parts))
        return ModelSpec(
            architecture=cfg.architecture, hidden_size=H, vocab_size=c["vocab_size"], max_position=256,
            embedding=PartSpec("token_embedding", {"vocab_size": c["vocab_size"], "hidden_size": H}, {"weight": ("emb",)}),
            layers=tuple(layers), run_order=tuple(RunEntry(i, i) for i in range(c["num_hidden_layers"])),
            final_norm=PartSpec("rmsnorm", {"size": H, "eps": c["eps"]}, {"weight": ("norm",)}),
            lm_head=PartSpec("lm_head", {"vocab_size": c["vocab_size"], "hidden_size": H, "tied": False},
                             {"weight": ("head",)}))

    register_architecture("ToySandwichLM", from_dict, build_spec)


_SANDWICH = {"architectures": ["ToySandwichLM"], "hidden_size": 48, "num_hidden_layers": 4, "vocab_size": 83,
             "inter": 56, "eps": 1e-5, "rank": 12, "heads": 3, "head_dim": 16, "grid_width": 5}


def _sandwich_plain(model_dir, tokens):
    """The toy architecture written out plainly: whole sequence, float64, no cache."""
    c = plain.read_config(model_dir)
    w = plain.read_tensors(model_dir)
    H, eps, r, nh, hd, gw = c["hidden_size"], c["eps"], c["rank"], c["heads"], c["head_dim"], c["grid_width"]
    T = len(tokens)
    pos = torch.arange(T)
    causal = pos[None, :] > pos[:, None]

    def grid_rotate(x):                                   # [T, heads, hd]
        half = hd // 2
        inv = 1.0 / (100.0 ** (torch.arange(0, half, 2, dtype=torch.float64) / half))
        out = x.clone()
        for sl, p in ((slice(0, half), pos // gw), (slice(half, hd), pos % gw)):
            ang = p.double()[:, None] * inv[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            a, b = x[..., sl][..., :half // 2], x[..., sl][..., half // 2:]
            out[..., sl] = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
        return out

    res = w["emb"][torch.as_tensor(tokens)]
    for i in range(c["num_hidden_layers"]):
        p = f"l{i}"
        a = plain.rms_norm(res, w[f"{p}.n1"], eps)
        if i % 2 == 0:
            q, lat = a @ w[f"{p}.wq"], a @ w[f"{p}.wc"]
            s = ((q @ lat.T) * r ** -0.5).masked_fill(causal, float("-inf"))
            m = (torch.softmax(s, dim=-1) @ lat) @ w[f"{p}.wo"].T
        else:
            q = plain.rms_norm((a @ w[f"{p}.q"].T).view(T, nh, hd), w[f"{p}.qn"], eps)
            k = plain.rms_norm((a @ w[f"{p}.k"].T).view(T, 1, hd), w[f"{p}.kn"], eps)
            v = (a @ w[f"{p}.v"].T).view(T, 1, hd)
            o = plain.causal_attention(grid_rotate(q), grid_rotate(k), v, hd ** -0.5)
            m = o.reshape(T, nh * hd) @ w[f"{p}.o"].T
        res = res + plain.rms_norm(m, w[f"{p}.n2"], eps)
        if i != 1:
            b = plain.rms_norm(res, w[f"{p}.n3"], eps)
            gu = torch.cat((b @ w[f"{p}.gate"].T, b @ w[f"{p}.up"].T), dim=-1)
            res = res + plain.rms_norm(plain.silu_and_mul(gu) @ w[f"{p}.down"].T, w[f"{p}.n4"], eps)
    return (plain.rms_norm(res, w["norm"], eps) @ w["head"].T).numpy()


def test_toy_arrangement_with_four_norms_latent_cache_rows_and_grid_positions(tmp_path):
    """Registered here, built from a random-weights folder and stepped through ModelRunner without a change
    to the package: an arrangement of its own (four norms; a layer without feed-forward), a mixer whose pages
    hold one 32-bit row per token beside attention layers whose pages hold keys and values (two page groups
    with block tables of their own), a parameter stacked side by side, and a position encoding applied
    between the mixer's norm and its cache write.  Portions beside single tokens, pages used again."""
    from atom_b200.config import EngineConfig, config_from_dict
    from atom_b200.engine.batch import StepEntry
    from atom_b200.engine.runner import ModelRunner
    from atom_b200.weights import write_random_model

    _register_sandwich()
    d = str(tmp_path / "sandwich")
    write_random_model(d, config_from_dict(_SANDWICH), seed=33)
    runner = ModelRunner(EngineConfig(model=d, dtype="float32", kv_cache_block_size=8, num_kvcache_blocks=10,
                                      max_num_seqs=3, enforce_eager=True))
    assert len(runner.cache.groups) == 2
    assert sorted(tuple(e.name for e in g.entries) for g in runner.cache.groups) == [("k", "v"), ("latent",)]
    rng = np.random.default_rng(5)
    seqs = {"x": rng.integers(0, 83, 37).tolist(), "y": rng.integers(0, 83, 22).tolist(),
            "z": rng.integers(0, 83, 30).tolist()}
    ref = {r: _sandwich_plain(d, t) for r, t in seqs.items()}
    got, done = {r: [] for r in seqs}, {r: 0 for r in seqs}
    # 10 pages of 8 tokens in each group: x (37) and y (22) hold 8, z (30) needs 4: two of them were y's
    plan = [{"x": 13}, {"x": 2, "y": 19}, {"x": 1, "y": 1}, {"x": 20, "y": 2}, {"x": 1, "z": 9}, {"z": 19}, {"z": 2}]
    for portions in plan:
        entries = [StepEntry(r, seqs[r][done[r]:done[r] + n], list(range(n))) for r, n in portions.items()]
        logits = runner.step(entries).cpu().numpy()
        o = 0
        for r, n in portions.items():
            got[r].append(logits[o:o + n])
            o += n
            done[r] += n
            if done[r] == len(seqs[r]):
                runner.finish(r)
    runner.check_status()
    runner.cache.check()
    for r in seqs:
        assert done[r] == len(seqs[r])
        err = np.abs(np.concatenate(got[r]) - ref[r]).max()
        assert err < 2e-4, f"{r}: max abs error {err:.2e}"
    assert all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
