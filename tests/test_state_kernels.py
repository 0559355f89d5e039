"""The kernels of the state mixers, of the normed and rotated attention inputs and of the weighted
residual sum, each alone against the plain functions of ``plain_fiferax`` (float64), over sizes that
take every cut of the scan (lanes a column, key channels a lane, columns a block, tokens a chunk)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_fiferax as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
PAGE = 64


def batch_of(lens, slots):
    """The fields of a step's batch that the kernels read: sequences packed one after the other."""
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)

    def i32(v):
        return torch.tensor(v, dtype=torch.int32, device=DEV)

    return SimpleNamespace(seq_starts=i32(starts), slots=i32(slots), n_seqs=len(lens), n_tokens=starts[-1])


def close(got, ref, tol=2e-5):
    ref = ref.double()
    err = float((got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
    assert err < tol, err


@pytest.mark.parametrize("heads,dk,dv", [(2, 8, 8), (3, 24, 40), (1, 32, 32), (2, 64, 16), (2, 100, 36),
                                         (1, 128, 128), (1, 200, 72), (1, 4, 4), (2, 6, 10)])
def test_delta_rule_scan(heads, dk, dv):
    """Two sequences in one step against the plain rule; then the longer one again in three steps of
    unequal sizes down to one token (the state is carried), in a slot that another sequence used before;
    a padding row (slot -1) changes nothing and leaves zeros."""
    from airframe_b200 import kernels
    lens = [37, 5]
    T = sum(lens)
    g = torch.Generator().manual_seed(dk * 131 + dv)
    r, k, v = (torch.randn(T, heads * n, generator=g) for n in (dk, dk, dv))
    w = torch.rand(T, heads * dk, generator=g) * 0.5 + 0.5
    a = torch.rand(T, heads * dk, generator=g)
    u = k.view(T, heads, dk) / torch.sqrt((k.view(T, heads, dk) ** 2).sum(-1, keepdim=True) + 1e-6)
    au = (a.view(T, heads, dk) * u).reshape(T, -1)
    ref, at = [], 0
    for n in lens:
        s = slice(at, at + n)
        o, S = plain.delta_rule(r[s].double().view(n, heads, dk), k[s].double().view(n, heads, dk),
                                v[s].double().view(n, heads, dv), w[s].double().view(n, heads, dk),
                                a[s].double().view(n, heads, dk))
        ref.append((o.reshape(n, -1), S))
        at += n
    state = torch.zeros(4, heads, dv, dk, device=DEV)
    dev = [t.to(DEV) for t in (r, k, v, w, u.reshape(T, -1), au)]
    out = torch.full((T, heads * dv), 7.0, device=DEV)
    kernels.state_scan("delta", out, dev[0], dev[1], dev[2], state, batch_of(lens, [2, 0]), heads, dk, dv,
                       w=dev[3], u=dev[4], au=dev[5])
    close(out[:37], ref[0][0])
    close(out[37:], ref[1][0])
    close(state[2].transpose(1, 2), ref[0][1])
    close(state[0].transpose(1, 2), ref[1][1])
    assert float(state[1].abs().sum()) == 0 and float(state[3].abs().sum()) == 0
    # the first sequence again, in portions, in the slot the second one used; a padding row rides along
    state[0].zero_()
    got = []
    at = 0
    for n in (19, 13, 2, 1, 2):
        rows = [t[at:at + n].contiguous() for t in dev]
        pad = [torch.cat([t, torch.ones(1, t.shape[1], device=DEV)]) for t in rows]
        o = torch.full((n + 1, heads * dv), 7.0, device=DEV)
        before = state.clone()
        kernels.state_scan("delta", o, pad[0], pad[1], pad[2], state, batch_of([n, 1], [0, -1]), heads, dk, dv,
                           w=pad[3], u=pad[4], au=pad[5])
        assert float(o[n].abs().sum()) == 0 and torch.equal(before[1:], state[1:])
        got.append(o[:n])
        at += n
    close(torch.cat(got), ref[0][0])
    close(state[0].transpose(1, 2), ref[0][1])


@pytest.mark.parametrize("heads,dk,dv", [(3, 8, 20), (2, 12, 12), (2, 32, 64), (1, 128, 128), (4, 16, 16), (1, 72, 8)])
def test_decay_scan_with_silu(heads, dk, dv):
    from airframe_b200 import kernels
    lens = [50, 1, 9]
    T = sum(lens)
    g = torch.Generator().manual_seed(dk + 7 * dv)
    q, k, v = (torch.randn(T, heads * n, generator=g) for n in (dk, dk, dv))
    decay = torch.tensor([1.0, 0.5, 0.97, 0.999][:heads])
    state = torch.zeros(3, heads, dv, dk, device=DEV)
    out = torch.empty(T, heads * dv, device=DEV)
    # q, k, v as sections of one wider row, as a packed projection gives them
    packed = torch.cat([q, torch.zeros(T, 3), k, v], dim=1).to(DEV)
    oq, ok, ov = 0, heads * dk + 3, 2 * heads * dk + 3
    kernels.state_scan("decay", out, packed[:, oq:oq + heads * dk], packed[:, ok:ok + heads * dk],
                       packed[:, ov:ov + heads * dv], state, batch_of(lens, [1, 2, 0]), heads, dk, dv,
                       decay=decay.to(DEV), silu=True)
    at = 0
    for n in lens:
        s = slice(at, at + n)
        ref = plain.decay_linear_attention(plain.silu(q[s].double()).view(n, heads, dk),
                                           plain.silu(k[s].double()).view(n, heads, dk),
                                           plain.silu(v[s].double()).view(n, heads, dv), decay.double())
        close(out[s], ref.reshape(n, -1))
        at += n


def test_delta_prep():
    from airframe_b200 import kernels
    T, heads, dk, rank = 9, 3, 20, 7
    n = heads * dk
    g = torch.Generator().manual_seed(1)
    proj = torch.randn(T, 2 * n + rank + 5, generator=g)
    off_k, off_a, off_w1 = 5, 5 + n, 5 + 2 * n
    a_bias, w0 = torch.randn(n, generator=g), torch.randn(n, generator=g)
    w2 = torch.randn(n, rank, generator=g)
    out = torch.empty(T, 3, n, device=DEV)
    kernels.delta_prep(out, proj.to(DEV), off_k, off_a, off_w1, a_bias.to(DEV), w0.to(DEV), w2.t().contiguous().to(DEV), heads, dk,
                       math.exp(-0.5), 1e-6)
    p = proj.double()
    k = p[:, off_k:off_k + n].view(T, heads, dk)
    u = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).reshape(T, n)
    w = torch.exp(-math.exp(-0.5) * plain.sigmoid(torch.tanh(p[:, off_w1:off_w1 + rank]) @ w2.double().T + w0.double()))
    a = plain.sigmoid(p[:, off_a:off_a + n] + a_bias.double())
    close(out[:, 0], w, 1e-6)
    close(out[:, 1], u, 1e-6)
    close(out[:, 2], a * u, 1e-6)


@pytest.mark.parametrize("width", [5, 44, 128, 300])
def test_gated_scan(width):
    from airframe_b200 import kernels
    lens = [23, 1, 6]
    T = sum(lens)
    g = torch.Generator().manual_seed(width)
    proj = torch.randn(T, 3 * width + 2, generator=g) * 2
    bz, bx = torch.randn(width, generator=g), torch.randn(width, generator=g)
    oz, ox, og = 2, 2 + width, 2 + 2 * width
    state = torch.zeros(5, width, device=DEV)
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        state.zero_()
        y = torch.empty(T, width, dtype=dt, device=DEV)
        kernels.gated_scan(y, proj.to(DEV), oz, ox, og, bz.to(DEV), bx.to(DEV), state, batch_of(lens, [4, 0, 2]))
        at = 0
        for n, slot in zip(lens, [4, 0, 2]):
            p = proj[at:at + n].double()
            z = plain.sigmoid(p[:, oz:oz + width] + bz.double())
            c = p[:, ox:ox + width] + bx.double()
            S = plain.gated_recurrence(z, torch.where(c >= 0, c + 0.5, plain.sigmoid(c)))
            close(y[at:at + n], S * plain.silu(p[:, og:og + width]), tol)
            close(state[slot], S[-1], 2e-6)
            at += n


@pytest.mark.parametrize("n,group", [(48, 24), (60, 60), (256, 128), (24, 8)])
def test_gated_group_norm(n, group):
    from airframe_b200 import kernels
    T = 7
    g = torch.Generator().manual_seed(n)
    o, w, gate = torch.randn(T, n, generator=g) * 3, torch.randn(n, generator=g), torch.randn(T, n + 4, generator=g)
    y = torch.empty(T, n, device=DEV)
    kernels.gated_group_norm(y, o.to(DEV), w.to(DEV), gate.to(DEV)[:, 4:], group, 1e-5)
    ref = plain.rms(o.double().view(T, n // group, group), 1e-5).reshape(T, n) * w.double() * plain.sigmoid(gate[:, 4:].double())
    close(y, ref, 2e-6)


@pytest.mark.parametrize("nq,nkv,hd,rot,shared_v", [(4, 4, 12, 6, True), (6, 2, 64, 64, True), (2, 1, 20, 0, True),
                                                    (3, 3, 16, 16, False)])
def test_norm_rotate_pack_and_store(nq, nkv, hd, rot, shared_v):
    """q and k heads normed and rotated, v taken from the raw k (or its own heads), rows packed, and k and v
    in the cache: a ring of 64 rows in which, of two tokens that share a row, the later one stays."""
    from airframe_b200 import kernels
    from airframe_b200.cache.sequence_cache import KVView
    from airframe_b200.parts.base import KVNeed
    lens = [70, 3]
    T = sum(lens)
    g = torch.Generator().manual_seed(hd)
    width_in = (nq + nkv + (0 if shared_v else nkv)) * hd
    proj = torch.randn(T, width_in, generator=g)
    qw, kw = torch.randn(hd, generator=g), torch.randn(hd, generator=g)
    inv = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32)
    pos = torch.tensor(list(range(70)) + list(range(3)), dtype=torch.int32, device=DEV)
    b = batch_of(lens, [1, 0])
    b.positions = pos
    b.seq_of_token = torch.tensor([0] * 70 + [1] * 3, dtype=torch.int32, device=DEV)
    b.len_after = torch.tensor(lens, dtype=torch.int32, device=DEV)
    kc = torch.zeros(4, nkv, PAGE, hd, device=DEV)
    vc = torch.zeros(4, nkv, PAGE, hd, device=DEV)
    table = torch.tensor([[3], [2]], dtype=torch.int32, device=DEV)            # slot -> its one page
    kv = KVView(kc, vc, table, PAGE, KVNeed(nkv, hd, 40))
    qkv = torch.empty(T, (nq + 2 * nkv) * hd, device=DEV)
    kernels.qk_norm_rope_store(qkv, proj.to(DEV), b, nq, nkv, hd, inv.to(DEV), rot, "half", q_weight=qw.to(DEV),
                               k_weight=kw.to(DEV), eps=1e-5, v_from_k=shared_v, kv=kv)
    p = proj.double()
    q = p[:, :nq * hd].view(T, nq, hd)
    k = p[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd)
    v = k if shared_v else p[:, (nq + nkv) * hd:].view(T, nkv, hd)
    positions = pos.cpu().long()
    qr = plain.rotate_half(plain.rms(q, 1e-5, qw.double()), positions, 50.0, rot)
    kr = plain.rotate_half(plain.rms(k, 1e-5, kw.double()), positions, 50.0, rot)
    close(qkv[:, :nq * hd], qr.reshape(T, -1), 3e-6)
    close(qkv[:, nq * hd:(nq + nkv) * hd], kr.reshape(T, -1), 3e-6)
    close(qkv[:, (nq + nkv) * hd:], v.reshape(T, -1), 1e-7)
    # sequence 0 (slot 1, page 2): rows 0..5 hold positions 64..69, rows 6..63 positions 6..63
    for row, t in [(0, 64), (5, 69), (6, 6), (63, 63)]:
        close(kc[2, :, row], kr[t], 3e-6)
        close(vc[2, :, row], v[t], 1e-7)
    close(kc[3, :, 2], kr[72], 3e-6)
    assert float(kc[3, :, 3:].abs().sum()) == 0 and float(kc[:2].abs().sum()) == 0


def test_weighted_residual_sum_and_norm():
    from airframe_b200 import kernels
    n, H = 11, 72
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(n, H, generator=g)
    a = torch.randn(n, H, generator=g).to(torch.bfloat16)
    parts = torch.randn(3, n, H, generator=g)
    w = torch.randn(H, generator=g)
    x = x0.to(DEV)
    y = torch.empty(n, H, device=DEV)
    kernels.add_scaled_rmsnorm(x, [(a.to(DEV), 0.8), (parts.to(DEV), 1.25)], y=y, w_next=w.to(DEV), eps=1e-5, offset=0.0)
    ref = x0.double() + 0.8 * a.double() + 1.25 * parts.double().sum(0)
    close(x, ref, 1e-6)
    close(y, plain.rms(ref, 1e-5, w.double()), 2e-6)
    x = x0.to(DEV)
    kernels.add_scaled_rmsnorm(x, [(parts.to(DEV), 1.0), (a.to(DEV), 1.0), (a.to(DEV), -1.0)])
    close(x, x0.double() + parts.double().sum(0), 1e-6)
