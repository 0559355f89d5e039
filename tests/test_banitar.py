"""Banitar through the engine against the plain implementation (``plain_banitar``): every way of
cutting the same requests into steps, in 32-bit and bfloat16, on configurations that differ in every
size, in the order of their layers, in where the repeated stretch lies and in their constants."""
import copy
import io
import json
import math

import pytest
import torch

import plain_banitar as plain
import replay
from tiny_banitar import BN_A, BN_B, CONFIGS, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

F64 = torch.float64


# ---------------------------------------------------------------- configuration (no GPU)

def test_config_round_trip_and_registry():
    from airframe_b200.config import BanitarConfig, config_from_dict
    cfg = config_from_dict(BN_A)
    assert isinstance(cfg, BanitarConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    spec = cfg.model_spec()
    kinds = [(layer.mixer.kind, layer.feed_forward.kind) for layer in spec.layers]
    assert kinds == [("latent_attention", "gated_mlp"), ("attention", "none"), ("attention", "gated_mlp"),
                     ("latent_attention", "none")]
    a = spec.layers[1].mixer.params
    assert a["mask"] == "chunk" and a["window"] == 7 and a["value_dim"] == 20 and a["position"].params["pairing"] == "adjacent"
    assert a["position"].params["scaling"]["factor"] == 4.0 and spec.layers[2].mixer.params["position"].params["scaling"] is None
    assert spec.layers[1].norms.keys() == {"pre_mixer", "post_mixer"}
    assert spec.layers[0].norms.keys() == {"pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward"}
    # the stretch 0..1 twice, entered through the junction each time with the number of the pass; then the rest
    assert [(e.layer, e.enter, e.enter_index) for e in spec.schedule] == \
        [(0, 0, 0), (1, None, 0), (0, 0, 1), (1, None, 0), (2, None, 0), (3, None, 0)]
    assert all(e.cache_from is None for e in spec.schedule)
    # no stretch: no junction, every layer once
    plain_cfg = copy.deepcopy(BN_A)
    plain_cfg.pop("loop")
    spec = config_from_dict(plain_cfg).model_spec()
    assert spec.junctions == [] and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    assert plain.layer_runs(BN_B) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert config_from_dict(BN_B).runs() == plain.layer_runs(BN_B)


def test_config_refuses_what_it_does_not_know():
    from airframe_b200.config import ConfigError, config_from_dict

    def broken(edit):
        d = copy.deepcopy(BN_A)
        edit(d)
        with pytest.raises(ConfigError):
            config_from_dict(d)

    broken(lambda d: d["layers"][0].update(type="convolution"))
    broken(lambda d: d["layers"][1]["mixer"].update(kv_heads=3))
    broken(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7))
    broken(lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14))
    broken(lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"))
    broken(lambda d: d["layers"][0]["mixer"]["rot"].update(dims=4))          # not the rotated part's size
    broken(lambda d: d["layers"][0]["mixer"].pop("kv_rank"))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="routed"))
    broken(lambda d: d["loop"].update(stop=5))
    broken(lambda d: d["loop"].update(times=0))
    broken(lambda d: d["loop"].update(start=2))
    broken(lambda d: d.pop("norm"))
    broken(lambda d: d["layers"][2]["mixer"]["mask"].pop("size"))


def test_declared_tensors():
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine.model import declared_weights
    decls = {d.name: tuple(d.shape) for d in declared_weights(config_from_dict(BN_A).model_spec())}
    assert decls["loop.in"] == (72, 144) and decls["loop.step"] == (2, 72)
    assert decls["l0.mix.q"] == (3 * 16, 72) and decls["l0.mix.dkv"] == (26, 72) and decls["l0.mix.dkv.norm"] == (20,)
    assert decls["l0.mix.uk"] == (30, 20) and decls["l0.mix.uv"] == (42, 20) and decls["l0.mix.o"] == (72, 42)
    assert decls["l0.mix.sink"] == (3,) and decls["l0.norm1.alpha"] == () and decls["l0.norm2b.b"] == (72,)
    assert decls["l1.mix.q"] == (48, 72) and decls["l1.mix.k.b"] == (24,) and decls["l1.mix.v"] == (40, 72)
    assert decls["l1.mix.g"] == (4, 72) and decls["l1.mix.o"] == (72, 80)
    assert "l1.norm2" not in decls and "l1.mlp.up" not in decls and "l0.mix.k" not in decls and "l1.mix.sink" not in decls
    assert decls["final.norm.alpha"] == () and decls["head"] == (211, 72)


# ---------------------------------------------------------------- the plain implementation on cases known by hand

def test_plain_masks_and_sink():
    w = plain.window_mask(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True] and w[1].tolist() == [True, True] + [False] * 4
    c = plain.chunk_mask(7, 3)
    assert c[5].tolist() == [False, False, False, True, True, True, False]
    assert c[3].tolist() == [False, False, False, True, False, False, False]      # the first of its chunk sees itself alone
    assert c[2].tolist() == [True, True, True, False, False, False, False]
    s = torch.zeros(2, 2, dtype=F64)
    p = plain.softmax_rows(s, plain.window_mask(2, 2), sink=torch.tensor(0.0, dtype=F64))
    assert torch.allclose(p, torch.tensor([[0.5, 0.0], [1 / 3, 1 / 3]], dtype=F64))   # the sink counts once, as exp(0)
    p = plain.softmax_rows(s, plain.window_mask(2, 2), sink=torch.tensor(math.log(2.0), dtype=F64))
    assert torch.allclose(p[1], torch.tensor([0.25, 0.25], dtype=F64))
    assert torch.allclose(plain.softmax_rows(s, plain.window_mask(2, 2)).sum(-1), torch.ones(2, dtype=F64))


def test_plain_rotations_and_frequencies():
    x = torch.randn(3, 1, 8, dtype=F64)
    pos = torch.tensor([0, 1, 2])
    one = torch.tensor(1.0, dtype=F64)
    f = plain.plain_frequencies(100.0, 4)
    assert f == [1.0, 100.0 ** -0.5]
    y = plain.rotate(x, pos, f, "half")
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])
    assert torch.allclose(y[1, 0, 0], x[1, 0, 0] * torch.cos(one) - x[1, 0, 2] * torch.sin(one))
    z = plain.rotate(x, pos, f, "adjacent", 2.0)
    assert torch.allclose(z[1, 0, 1], 2.0 * (x[1, 0, 1] * torch.cos(one) + x[1, 0, 0] * torch.sin(one)))
    assert torch.allclose(z[1, 0, 2], 2.0 * (x[1, 0, 2] * torch.cos(0.1 * one) - x[1, 0, 3] * torch.sin(0.1 * one)))
    # base 100, 8 dims, trained for 2 pi 10 positions: a pair turns 10 / 100^(i/4) times there; the pairs that turn
    # at least `fast` = 2 times keep their frequency, those that turn at most `slow` = 0.5 times are divided by 4
    s = {"factor": 4.0, "original": 2.0 * math.pi * 10.0, "fast": 2.0, "slow": 0.5}
    got, mag = plain.stretched_frequencies(100.0, 8, s)
    base = plain.plain_frequencies(100.0, 8)
    lo, hi = math.floor(8 * math.log(5.0) / (2 * math.log(100.0))), math.ceil(8 * math.log(20.0) / (2 * math.log(100.0)))
    assert (lo, hi) == (1, 3)
    assert got[0] == base[0] and got[1] == base[1] and abs(got[3] - base[3] / 4.0) < 1e-15
    assert abs(got[2] - (0.5 * base[2] / 4.0 + 0.5 * base[2])) < 1e-15
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    n = plain.unit_rms(torch.tensor([3.0, 4.0], dtype=F64), 0.0)
    assert torch.allclose(n, torch.tensor([3.0, 4.0], dtype=F64) / math.sqrt(12.5))


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
    the differences against that of the logits, and a looser bound on the largest one."""
    if dtype == "float32":
        assert rel_err(got, ref) < VS_PLAIN[dtype], what
        return
    assert rms_rel(got, ref) < rms, what
    assert rel_err(got, ref) < worst, what


def case(name, tmp_path_factory, edit=None, key=None, cfg_edit=None):
    """Folder, plain configuration and weights of a configuration (made once a session)."""
    key = key or name
    if key not in _CASES:
        cfg_dict = copy.deepcopy(CONFIGS[name])
        if cfg_edit is not None:
            cfg_edit(cfg_dict)
        folder = make_folder(cfg_dict, seed=11 + len(_CASES), root=tmp_path_factory.mktemp("bn" + key), edit=edit)
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
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    """A prompt in one step; the same tokens with the last 40 one by one (the captured decode step);
    and a prompt of one token followed by single tokens only (the first tokens of a sequence, decoded)."""
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
    agrees(replay.run_whole(rt, ids[:1]), ref[:1], dtype)


@gpu
@pytest.mark.parametrize("name", ["A", "B", "D", "F"])
def test_unequal_batches_and_slots_used_again(name, dtype, tmp_path_factory):
    """Requests of unequal lengths (one of a single token, one longer than its windows) in batches, then
    decoded together, the shorter ones leaving; twice, so that slots and pages are used again."""
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
    """Three tokens of prompt, then 290 single tokens: cache pages begin at 64, 128, 192 and 256; the window of
    130 and the chunks of 70 and 128 pass over decoded tokens, and their rings of 192 and 128 rows wrap."""
    c = case("B", tmp_path_factory)
    rt = load(c, dtype)
    ids = replay.random_ids(c["cfg"]["vocab"], 293, 9)
    agrees(replay.run_tail(rt, ids, 290), reference(c, ids), dtype)


def _sharp(cfg):
    """Scores four times as large: the softmax picks few keys, so a key that is wrongly seen or missed moves
    the logits by far more than rounding does."""
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] *= 4.0


def _loud_latent(name, t):
    """Queries and keys of the latent attention large enough for its scores to matter beside its sink."""
    if name.endswith("mix.uk") or name in ("l0.mix.q", "l3.mix.q"):            # (the latent layers of configuration A)
        return t * 4.0
    return t


@gpu
def test_window_and_chunk_edges_show(dtype, tmp_path_factory):
    c = case("A", tmp_path_factory, edit=_loud_latent, key="A-sharp", cfg_edit=_sharp)
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 60, 21)
    ref = reference(c, ids)
    # the plain implementation with a window or a chunk one token off gives other logits, well beyond the tolerance
    for kind in ("attention", "latent_attention"):
        for delta in (-1, 1):
            off = copy.deepcopy(cfg)
            for layer in off["layers"]:
                if layer["type"] == kind:
                    layer["mixer"]["mask"]["size"] += delta
            wrong = plain.logits(off, w, ids)
            assert rms_rel(wrong, ref) > 0.05, (kind, delta)
    # chunks counted from where the prompt was cut instead of from position 0 would show as well
    rt = load(c, dtype)
    agrees(replay.run_whole(rt, ids), ref, dtype, rms=0.06, worst=0.3)
    agrees(replay.run_tail(rt, ids, 50), ref, dtype, rms=0.06, worst=0.3)
    agrees(replay.run_tail(rt, ids, 17), ref, dtype, rms=0.06, worst=0.3)


@gpu
def test_sink_and_gate_and_norm_after_rotation_show(dtype, tmp_path_factory):
    """Leaving out the sink, the output gate, the biases or the norm after the rotation moves the plain logits far
    beyond the tolerance that the engine keeps."""
    c = case("A", tmp_path_factory, edit=_loud_latent, key="A-loud")
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 50, 8)
    ref = reference(c, ids)
    no_sink = {k: (torch.full_like(v, -1e30) if k.endswith(".sink") else v) for k, v in w.items()}
    assert rms_rel(plain.logits(cfg, no_sink, ids), ref) > 0.04
    open_gate = {k: (torch.zeros_like(v) if k.endswith("mix.g") else v) for k, v in w.items()}
    assert rms_rel(plain.logits(cfg, open_gate, ids), ref) > 0.04
    no_bias = {k: (torch.zeros_like(v) if k.endswith(("mix.q.b", "mix.k.b", "mix.v.b")) else v) for k, v in w.items()}
    assert rms_rel(plain.logits(cfg, no_bias, ids), ref) > 0.04
    rt = load(c, dtype)
    agrees(replay.run_whole(rt, ids), ref, dtype)
    agrees(replay.run_tail(rt, ids, 30), ref, dtype)


@gpu
def test_far_tokens_show(dtype, tmp_path_factory):
    """The first token reaches the last logits through the chain of layers alone (every window and chunk is
    far shorter than the prompt) and through the embedding's output that every pass through the stretch takes in;
    the second through the layers only."""
    c = case("B", tmp_path_factory)
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 260, 33)
    ref = reference(c, ids)
    other = ids[:200] + [(ids[200] + 1) % cfg["vocab"]] + ids[201:]        # 59 tokens back: beyond the short window's reach
    assert rel_err(plain.logits(cfg, w, other)[-1:], ref[-1:]) > 10 * VS_PLAIN["float32"]
    first = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]                       # 259 back: beyond every window, and felt all the same
    assert rel_err(plain.logits(cfg, w, first)[-1:], ref[-1:]) > 3 * VS_PLAIN["float32"]
    rt = load(c, dtype)
    agrees(replay.run_tail(rt, ids, 8)[-8:], ref[-8:], dtype)
    agrees(replay.run_whole(rt, ids)[-8:], ref[-8:], dtype)


@gpu
def test_layers_agree_one_by_one(tmp_path_factory):
    """The residual stream after every run of a layer, 32-bit, against the plain implementation's."""
    from airframe_b200.engine import StepEntry

    class Keep:
        def __init__(self):
            self.x = []

        def after(self, run, layer, x, batch):
            if run >= 0:
                self.x.append(x.detach().cpu().double())

    for name in ("A", "B", "C", "D", "E", "F"):
        c = case(name, tmp_path_factory)
        rt = load(c, "float32")
        ids = replay.random_ids(c["cfg"]["vocab"], 75, 2)
        per_run = plain.residual_streams(c["cfg"], c["w"], ids)
        s = rt.engine.take_slot()
        keep = Keep()
        rt.engine.step([StepEntry(s, ids, [0])], probe=keep)
        rt.engine.free_slot(s)
        assert len(keep.x) == len(per_run)
        for i, (got, ref) in enumerate(zip(keep.x, per_run)):
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
def test_trace_replay_of_a_banitar_folder(tmp_path, tmp_path_factory):
    from airframe_b200.cli.trace_run import main
    c = case("D", tmp_path_factory)
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
    """The named small configuration on a prompt of 2,500 tokens that laps its rings many times, then 70 single
    tokens: too long for the plain implementation, so the engine is held against itself: the 32-bit logits must
    not depend on where the prompt ends and the single tokens begin, and bfloat16 must agree with 32-bit within
    its rounding."""
    from airframe_b200.config.presets import preset
    folder = make_folder(preset("banitar-small"), seed=4, root=tmp_path_factory.mktemp("bnsmall"))
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
