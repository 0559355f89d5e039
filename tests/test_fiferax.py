"""Fiferax through the engine against the plain implementation (``plain_fiferax``): every way of
cutting the same requests into steps, in 32-bit and bfloat16, on configurations that differ in every
size, in the order of their layers and in their constants."""
import copy
import io
import json

import pytest
import torch

import plain_fiferax as plain
import replay
from tiny_fiferax import CONFIGS, FX_A, FX_B, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err


# ---------------------------------------------------------------- configuration (no GPU)

def test_config_round_trip_and_registry():
    from airframe_b200.config import FiferaxConfig, config_from_dict
    cfg = config_from_dict(FX_A)
    assert isinstance(cfg, FiferaxConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    spec = cfg.model_spec()
    kinds = [(layer.mixer.kind, layer.feed_forward.kind) for layer in spec.layers]
    assert kinds == [("parallel", "gated_mlp"), ("general_delta", "none"), ("mingru", "gated_mlp"),
                     ("general_delta", "gated_mlp"), ("parallel", "none")]
    left = spec.layers[4].mixer.params["branches"][0]
    assert left["scale"] == 0.6 and left["mixer"].params["window"] == 9 and left["mixer"].params["v_weight"] is None
    assert spec.layers[1].norms.keys() == {"pre_mixer"}


def test_config_refuses_what_it_does_not_know():
    from airframe_b200.config import ConfigError, config_from_dict

    def broken(edit):
        d = copy.deepcopy(FX_A)
        edit(d)
        with pytest.raises(ConfigError):
            config_from_dict(d)

    broken(lambda d: d["layers"][0].update(type="convolution"))
    broken(lambda d: d["layers"][0]["mixer"]["left"].update(vdim=16))
    broken(lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5]))
    broken(lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3))
    broken(lambda d: d["layers"][2]["mlp"].update(kind="routed"))
    broken(lambda d: d.pop("norm"))
    broken(lambda d: d["layers"][1]["mixer"].pop("dim"))


def test_declared_tensors_and_the_rank_from_the_file(tmp_path):
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine.model import declared_weights
    from airframe_b200.weights.loader import shape_fits
    decls = {d.name: d for d in declared_weights(config_from_dict(FX_A).model_spec())}
    assert decls["l1.mix.w1"].shape == (5, 72) and decls["l1.mix.w2"].shape == (48, 5)
    assert decls["l0.mix.left.q.norm"].shape == (12,) and "l0.mix.left.v" not in decls
    assert decls["l0.mix.right.v"].shape == (60, 72) and "l1.norm2" not in decls and "l0.norm2" in decls
    # without the key, the rank is whatever the stored tensor has
    d = copy.deepcopy(FX_A)
    d["layers"][1]["mixer"].pop("rank")
    open_decls = {x.name: x for x in declared_weights(config_from_dict(d).model_spec())}
    assert open_decls["l1.mix.w1"].shape == (None, 72)
    assert shape_fits((None, 72), (9, 72)) and not shape_fits((None, 72), (9, 71)) and not shape_fits((None,), (9, 72))


# ---------------------------------------------------------------- the plain implementation on cases known by hand

def test_plain_delta_rule_known_cases():
    T, H, d = 5, 1, 3
    g = torch.Generator().manual_seed(3)
    r, k, v = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for _ in range(3))
    one, zero = torch.ones(T, H, d, dtype=torch.float64), torch.zeros(T, H, d, dtype=torch.float64)
    # no decay, nothing removed: plain linear attention
    o, _ = plain.delta_rule(r, k, v, one, zero)
    lin = plain.decay_linear_attention(r, k, v, torch.ones(H, dtype=torch.float64))
    assert torch.allclose(o, lin)
    # the same unit key written twice with full removal: the second value replaces the first
    k2 = torch.tensor([[[1.0, 0.0, 0.0]], [[1.0, 0.0, 0.0]]], dtype=torch.float64)
    v2 = torch.tensor([[[1.0, 2.0, 3.0]], [[7.0, 8.0, 9.0]]], dtype=torch.float64)
    o2, S = plain.delta_rule(k2, k2, v2, one[:2], one[:2], key_eps=0.0)
    assert torch.allclose(S[0, 0], v2[1, 0]) and torch.allclose(o2[1, 0], v2[1, 0])


def test_plain_small_pieces():
    z = torch.ones(4, 2, dtype=torch.float64)
    c = torch.arange(8, dtype=torch.float64).view(4, 2)
    assert torch.equal(plain.gated_recurrence(z, c), c)                     # gate open: the candidate
    assert torch.allclose(plain.gated_recurrence(z * 0.5, c)[1], 0.5 * (0.5 * c[0]) + 0.5 * c[1])
    q = torch.randn(6, 2, 4, dtype=torch.float64)
    kv = torch.randn(6, 1, 4, dtype=torch.float64)
    assert torch.allclose(plain.windowed_attention(q, kv, kv, 0.3, 1), kv.expand(6, 2, 4))   # sees itself alone
    x = torch.randn(3, 1, 8, dtype=torch.float64)
    y = plain.rotate_half(x, torch.tensor([0, 1, 2]), 100.0, 4)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])
    assert torch.allclose(y[1, 0, 0], x[1, 0, 0] * torch.cos(torch.tensor(1.0, dtype=torch.float64))
                          - x[1, 0, 2] * torch.sin(torch.tensor(1.0, dtype=torch.float64)))
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12


# ---------------------------------------------------------------- the engine

gpu = pytest.mark.gpu


@pytest.fixture(params=["float32", "bfloat16"])
def dtype(request):
    return request.param


_CASES = {}


def rms_rel(got, ref) -> float:
    d = got.double().cpu() - ref.double()
    return float(d.pow(2).mean().sqrt() / ref.double().pow(2).mean().sqrt())


def agrees(got, ref, dtype, what=None, rms=3e-2, worst=0.15):
    """32-bit: the largest difference against the largest reference logit.  bfloat16: the root mean square of
    the differences against that of the logits, and a looser bound on the largest one: the first tokens of a
    sequence divide nearly empty states by their own size (a head's output at position 0 is its value times
    the scalar r.k, of which the norm keeps the sign alone), so single rows carry more rounding than the rest."""
    if dtype == "float32":
        assert rel_err(got, ref) < VS_PLAIN[dtype], what
        return
    assert rms_rel(got, ref) < rms, what
    assert rel_err(got, ref) < worst, what


def case(name, tmp_path_factory, edit=None, key=None):
    """Folder, plain configuration and weights of a configuration (made once a session)."""
    key = key or name
    if key not in _CASES:
        folder = make_folder(CONFIGS[name], seed=11 + len(_CASES), root=tmp_path_factory.mktemp("fx" + key), edit=edit)
        cfg, w = plain.read_model_folder(folder)
        _CASES[key] = {"folder": folder, "cfg": cfg, "w": w, "ref": {}}
    return _CASES[key]


def reference(c, ids):
    k = tuple(ids)
    if k not in c["ref"]:
        c["ref"][k] = plain.logits(c["cfg"], c["w"], ids)
    return c["ref"][k]


def load(c, dtype, max_tokens=64 * 24, **kw):
    from airframe_b200.engine import GpuRuntime
    return GpuRuntime.load(c["folder"], dtype=dtype, max_tokens=max_tokens, **kw)


@gpu
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    """A prompt in one step; the same tokens with the last 40 one by one (the captured decode step);
    and a prompt of one token followed by single tokens only."""
    c = case(name, tmp_path_factory)
    rt = load(c, dtype)
    ids = replay.random_ids(c["cfg"]["vocab"], 150, 5)
    ref = reference(c, ids)
    whole = replay.run_whole(rt, ids)
    agrees(whole, ref, dtype)
    tail = replay.run_tail(rt, ids, 40)
    agrees(tail, ref, dtype)
    if dtype == "float32":
        assert rel_err(tail, whole) < SPLITS[dtype] * 4
    short = ids[:70]
    agrees(replay.run_tail(rt, short, 69), ref[:70], dtype)


@gpu
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_unequal_batches_and_slots_used_again(name, dtype, tmp_path_factory):
    """Requests of unequal lengths (one of a single token, one longer than its windows) in batches, then
    decoded together, the shorter ones leaving; twice, so that slots, pages and states are used again."""
    c = case(name, tmp_path_factory)
    rt = load(c, dtype)
    V = c["cfg"]["vocab"]
    reqs = [replay.random_ids(V, n, 100 + n) for n in (90, 1, 37, 160, 66, 12)]
    refs = [reference(c, r) for r in reqs]
    prompt_lens = [70, 1, 5, 150, 64, 2]
    seen = []
    for rnd in range(2):
        out, slots = replay.run_batches(rt, reqs, 4, prompt_lens)
        seen.append(slots)
        for i, r in enumerate(refs):
            agrees(out[i], r, dtype, (rnd, i))
    assert seen[0] == seen[1]                      # the same slots served other requests in between
    # each alone gives what it gave in company
    alone = replay.run_tail(rt, reqs[3], 10)
    if dtype == "float32":
        assert rel_err(alone, out[3]) < SPLITS[dtype] * 4
    else:
        agrees(alone, refs[3], dtype)


@gpu
def test_long_decoding_over_pages_and_rings(dtype, tmp_path_factory):
    """Three tokens of prompt, then 230 single tokens: cache pages begin at 64, 128 and 192, the windows of 70
    and 130 tokens pass over decoded tokens, and their rings of 128 and 192 rows wrap."""
    c = case("B", tmp_path_factory)
    rt = load(c, dtype)
    ids = replay.random_ids(c["cfg"]["vocab"], 233, 9)
    agrees(replay.run_tail(rt, ids, 230), reference(c, ids), dtype)


def _peaky(name, t):
    """Query and key norms six times as large: the softmax picks few keys, so a key that is wrongly seen or
    missed moves the logits by far more than rounding does."""
    return t * 6.0 if name.endswith("q.norm") or name.endswith("k.norm") else t


@gpu
def test_window_edges_show(dtype, tmp_path_factory):
    c = case("A", tmp_path_factory, edit=_peaky, key="A-peaky")
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 40, 21)
    ref = reference(c, ids)
    # the plain implementation with windows one token off gives other logits, well beyond the tolerance
    for delta in (-1, 1):
        off = copy.deepcopy(cfg)
        for layer in off["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["left"]["mask"]["size"] += delta
        wrong = plain.logits(off, w, ids)
        assert rel_err(wrong, ref) > 0.5 and rms_rel(wrong, ref) > 0.4
    # (scores 36 times as large carry 36 times the rounding of bfloat16 queries and keys: its bound is looser
    # here, and still several times below what a window that is one token off does)
    rt = load(c, dtype)
    agrees(replay.run_whole(rt, ids), ref, dtype, rms=0.1, worst=0.4)
    agrees(replay.run_tail(rt, ids, 30), ref, dtype, rms=0.1, worst=0.4)


@gpu
def test_far_tokens_show(dtype, tmp_path_factory):
    """The first token reaches the last logits through the states alone (every window is shorter than the
    prompt): with a decay of 1 nothing of it is lost, and the plain implementation shows how much it matters."""
    c = case("A", tmp_path_factory)
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 120, 33)
    ref = reference(c, ids)
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    assert rel_err(plain.logits(cfg, w, other)[-8:], ref[-8:]) > 0.1
    rt = load(c, dtype)
    agrees(replay.run_tail(rt, ids, 8)[-8:], ref[-8:], dtype)
    agrees(replay.run_whole(rt, ids)[-8:], ref[-8:], dtype)


@gpu
def test_layers_agree_one_by_one(tmp_path_factory):
    """The residual stream after every layer, 32-bit, against the plain implementation's."""
    from airframe_b200.engine import StepEntry

    class Keep:
        def __init__(self):
            self.x = []

        def after(self, run, layer, x, batch):
            if run >= 0:
                self.x.append(x.detach().cpu().double())

    for name in ("A", "B", "C", "D"):
        c = case(name, tmp_path_factory)
        rt = load(c, "float32")
        ids = replay.random_ids(c["cfg"]["vocab"], 75, 2)
        per_layer = []
        plain.hidden_states(c["cfg"], c["w"], ids, per_layer)
        s = rt.engine.take_slot()
        keep = Keep()
        rt.engine.step([StepEntry(s, ids, [0])], probe=keep)
        rt.engine.free_slot(s)
        assert len(keep.x) == len(per_layer)
        for i, (got, ref) in enumerate(zip(keep.x, per_layer)):
            assert rel_err(got, ref) < 2e-5, (name, i)


@gpu
def test_greedy_generation_through_the_runtime(tmp_path_factory):
    from airframe_b200.sampling import SamplingParams
    c = case("A", tmp_path_factory)
    rt = load(c, "float32")
    V = c["cfg"]["vocab"]
    prompts = [replay.random_ids(V, n, 60 + n) for n in (9, 1, 30)]
    params = SamplingParams(max_tokens=12, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    got = rt.generate(prompts, params)
    want = [plain.generate_greedy(c["cfg"], c["w"], p, 12) for p in prompts]
    assert got == want
    assert rt.generate(prompts[2], params) == want[2]
    rt16 = load(c, "bfloat16")
    out = rt16.generate(prompts, params)
    assert [len(o) for o in out] == [12, 12, 12]


@gpu
def test_trace_replay_of_a_fiferax_folder(tmp_path, tmp_path_factory):
    from airframe_b200.cli.trace_run import main
    c = case("A", tmp_path_factory)
    V = c["cfg"]["vocab"]
    a, b = replay.random_ids(V, 20, 1), replay.random_ids(V, 7, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:18], "want": [0, 17]},
                                     {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[18]], "want": [0]},
                                     {"id": "b", "tokens": [b[6]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[19]], "want": []}], "end": ["a"]}]
    out = io.StringIO()
    code = main(["--model", str(c["folder"]), "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out)
    assert code == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    import numpy as np
    ra, rb = reference(c, a), reference(c, b)
    s0 = torch.from_numpy(np.fromfile(tmp_path / "0.f32", dtype="<f4")).view(2, V)
    s1 = torch.from_numpy(np.fromfile(tmp_path / "1.f32", dtype="<f4")).view(2, V)
    assert rel_err(s0, ra[[0, 17]]) < VS_PLAIN["float32"]
    assert rel_err(s1, torch.stack([ra[18], rb[6]])) < VS_PLAIN["float32"]
    assert not (tmp_path / "2.f32").exists()


@gpu
def test_long_prompt_at_layer_sizes_beyond_the_plain_implementation(tmp_path_factory):
    """The named small configuration (width 512, head size 64, a window of 256) on a prompt of 2,500 tokens
    that laps the window's ring ten times, then 70 single tokens: too long for the plain implementation, so
    the engine is held against itself: the 32-bit logits must not depend on where the prompt ends and the
    single tokens begin, and bfloat16 must agree with 32-bit within its rounding."""
    from airframe_b200.config.presets import preset
    from tiny_fiferax import make_folder as make
    folder = make(preset("fiferax-small"), seed=4, root=tmp_path_factory.mktemp("fxsmall"))
    from airframe_b200.engine import GpuRuntime, StepEntry
    ids = replay.random_ids(8192, 2570, 17)
    want = [0, 1, 255, 256, 257, 1023, 2047, 2499]

    def run(dtype, cut):
        rt = GpuRuntime.load(folder, dtype=dtype, max_tokens=64 * 48, max_context=4096)
        s = rt.engine.take_slot()
        out = [rt.step([StepEntry(s, ids[:cut], [w for w in want if w < cut])]).cpu()]
        for t in ids[cut:]:
            out.append(rt.step([StepEntry(s, [t], [0])]).cpu())
        rt.engine.free_slot(s)
        return torch.cat(out)

    a = run("float32", 2500)
    assert torch.isfinite(a).all()
    b = run("float32", 2540)
    # the last 30 tokens were single tokens in both runs; tokens 2500..2539 single in one, of the prompt in the other
    assert rel_err(b[-30:], a[-30:]) < 1e-4
    c = run("bfloat16", 2500)
    assert rms_rel(c, a) < 3e-2
