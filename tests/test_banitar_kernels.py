"""The kernels behind Banitar's mechanisms, each alone against the plain implementation's functions:
the norm without statistics and its fusions, the re-entry's sums, projections packed with biases, rotation and a
norm behind it, the latent rows, the small product per head, and attention with windows, chunks, sinks,
gates, values of another size than the keys and values that lie inside the key rows - prompts and single
tokens over a paged ring, on the plain kernels and on the tensor-core ones."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_banitar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
PAGE = 64


@pytest.fixture(scope="module")
def K():
    from airframe_b200 import kernels
    return kernels


def close(got, ref, tol):
    ref = ref.double().cpu()
    err = float((got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
    assert err < tol, err


def step_batch(lens, device=DEV, decode_from=None):
    """What the kernels read of a step: a prompt of each length, or (decode_from: lengths before) one token each."""
    pos, seq = [], []
    for b, n in enumerate(lens):
        if decode_from is None:
            pos += list(range(n))
            seq += [b] * n
        else:
            pos.append(decode_from[b])
            seq.append(b)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    after = lens if decode_from is None else [n + 1 for n in decode_from]
    starts = [0]
    for n in (lens if decode_from is None else [1] * len(lens)):
        starts.append(starts[-1] + n)
    return SimpleNamespace(positions=i32(pos), seq_of_token=i32(seq), slots=i32(list(range(len(lens)))),
                           len_after=i32(after), seq_starts=i32(starts), seq_lens=list(lens), n_seqs=len(lens),
                           max_len=max(lens), max_len_after=max(after), is_prefill=decode_from is None, aux={},
                           tokens=i32([0] * len(pos)), n_tokens=len(pos))


# ---------------------------------------------------------------- the norm and the re-entry

@pytest.mark.parametrize("H", [72, 51])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_tanh_norm_alone_and_fused(K, H, out_dtype):
    T = 37
    x = torch.randn(T, H, device=DEV) * 2
    w, b, w2, b2 = (torch.randn(H, device=DEV) for _ in range(4))
    tol = 1e-6 if out_dtype == torch.float32 else 5e-3
    y = torch.empty(T, H, dtype=out_dtype, device=DEV)
    K.tanh_norm(y, x, w, b, 0.7)
    close(y, torch.tanh(0.7 * x.double()) * w.double() + b.double(), tol)
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=DEV)
    y3 = torch.empty(3, H, dtype=out_dtype, device=DEV)
    K.tanh_norm(y3, x, w, b, -1.3, rows)
    close(y3, torch.tanh(-1.3 * x[rows.long()].double()) * w.double() + b.double(), tol)
    # x += norm(a), with a as it comes (the compute dtype, 32-bit, or partial sums), and the next norm of the new x
    for a in (torch.randn(T, H, device=DEV), torch.randn(T, H, device=DEV).bfloat16(), torch.randn(3, T, H, device=DEV)):
        x1 = x.clone()
        total = a.double().sum(0) if a.dim() == 3 else a.double()
        want = x.double() + torch.tanh(0.4 * total) * w.double() + b.double()
        y = torch.empty(T, H, dtype=out_dtype, device=DEV)
        K.add_tanh_norm(x1, a, w, b, 0.4, y=y, w_next=w2, b_next=b2, alpha_next=1.1)
        close(x1, want, 1e-6)
        close(y, torch.tanh(1.1 * want) * w2.double() + b2.double(), tol)
        x2 = x.clone()
        K.add_tanh_norm(x2, a, w, b, 0.4)
        assert torch.equal(x1, x2)


@pytest.mark.parametrize("H", [50, 72])
def test_reentry_sums(K, H):
    T = 19
    x, x0 = torch.randn(T, H, device=DEV), torch.randn(T, H, device=DEV)
    for dt in (torch.float32, torch.bfloat16):
        both = torch.empty(T, 2 * H, dtype=dt, device=DEV)
        K.concat_cast(both, x, x0)
        assert torch.equal(both, torch.cat([x, x0], 1).to(dt))
    z, row = torch.randn(4, T, H, device=DEV), torch.randn(H, device=DEV)
    w, b = torch.randn(H, device=DEV), torch.randn(H, device=DEV)
    out, y = torch.empty(T, H, device=DEV), torch.empty(T, H, device=DEV)
    K.set_sum_row(out, z, row, y=y, w=w, b=b, alpha=0.9)
    want = z.double().sum(0) + row.double()
    close(out, want, 1e-6)
    close(y, torch.tanh(0.9 * want) * w.double() + b.double(), 1e-6)
    K.set_sum_row(out, z[0].contiguous(), row)
    close(out, z[0].double() + row.double(), 1e-7)


# ---------------------------------------------------------------- projections packed for the attention kernels

def paged(n_pages, nkv, width, dtype):
    return torch.zeros(n_pages, nkv, PAGE, width, dtype=dtype, device=DEV)


def kv_view(k, v, table, ring):
    return SimpleNamespace(k=k, v=v, page_table=table, ring_rows=ring)


@pytest.mark.parametrize("nq,nkv,hd,dv,rot,pairing", [(4, 2, 12, 20, 8, "adjacent"), (3, 3, 64, 64, 64, "adjacent"),
                                                      (2, 1, 10, 6, 2, "half"), (6, 2, 64, 32, 32, "adjacent")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_rotation_norm_behind_it_and_store(K, nq, nkv, hd, dv, rot, pairing, dtype):
    lens = [70, 3]
    T = sum(lens)
    batch = step_batch(lens)
    width = (nq + nkv) * hd + nkv * dv
    proj = torch.randn(T, width + nq, device=DEV)              # (the gate's logits ride behind and are left alone)
    bias = torch.randn(width, device=DEV)
    freqs, mag = plain.stretched_frequencies(500.0, rot, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0})
    inv = torch.tensor(freqs, dtype=torch.float32, device=DEV)
    kc, vc = paged(5, nkv, hd, dtype), paged(5, nkv, dv, dtype)
    table = torch.tensor([[3, 1], [4, -1]], dtype=torch.int32, device=DEV)
    qkv = torch.empty(T, width, dtype=dtype, device=DEV)
    eps = 1e-5
    K.qk_norm_rope_store(qkv, proj, batch, nq, nkv, hd, inv, rot, pairing, eps=eps, kv=kv_view(kc, vc, table, 0),
                         bias=bias, norm_after=True, magnitude=mag, dv=dv)
    full = (proj[:, :width].double() + bias.double()).cpu()
    pos = batch.positions.cpu()
    q = plain.unit_rms(plain.rotate(full[:, : nq * hd].view(T, nq, hd), pos, freqs, pairing, mag), eps)
    k = plain.unit_rms(plain.rotate(full[:, nq * hd: (nq + nkv) * hd].view(T, nkv, hd), pos, freqs, pairing, mag), eps)
    v = full[:, (nq + nkv) * hd:].view(T, nkv, dv)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    close(qkv[:, : nq * hd], q.reshape(T, -1), tol)
    close(qkv[:, nq * hd: (nq + nkv) * hd], k.reshape(T, -1), tol)
    close(qkv[:, (nq + nkv) * hd:], v.reshape(T, -1), tol)
    # the cache: token 69 of the first sequence lies in its second page (3, then 1) at row 5; the second sequence in page 4
    close(kc[1, :, 5], k[69], tol)
    close(vc[1, :, 5], v[69], tol)
    close(kc[3, :, 63], k[63], tol)
    close(vc[4, :, 2], v[72], tol)
    assert float(kc[0].abs().max()) == 0 and float(kc[2].abs().max()) == 0       # nobody's pages stay untouched


@pytest.mark.parametrize("heads,dim,rot,rank,pitch", [(3, 10, 6, 20, 0), (2, 64, 16, 112, 128), (1, 5, 4, 11, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_rows_and_the_product_per_head(K, heads, dim, rot, rank, pitch, dtype):
    lens = [5, 66]
    T = sum(lens)
    batch = step_batch(lens)
    proj = torch.randn(T, heads * (dim + rot) + rank + rot, device=DEV)
    norm_w = torch.randn(rank, device=DEV)
    freqs = plain.plain_frequencies(77.0, rot)
    inv = torch.tensor(freqs, dtype=torch.float32, device=DEV)
    kc = paged(4, 1, rank + rot, dtype)
    table = torch.tensor([[2, -1], [0, 3]], dtype=torch.int32, device=DEV)
    P = pitch or dim + rot
    q = torch.full((T, heads * P), float("nan"), dtype=dtype, device=DEV)
    kvrow = torch.empty(T, rank + rot, dtype=dtype, device=DEV)
    K.latent_prep(q, kvrow, proj, batch, heads, dim, rot, rank, norm_w, 1e-5, inv, kv=kv_view(kc, None, table, 0), pitch=pitch)
    x = proj.double().cpu()
    pos = batch.positions.cpu()
    qh = x[:, : heads * (dim + rot)].view(T, heads, dim + rot)
    q_ref = torch.cat([qh[..., :dim], plain.rotate(qh[..., dim:], pos, freqs, "half")], -1)
    lat = x[:, heads * (dim + rot):]
    c = plain.unit_rms(lat[:, :rank], 1e-5) * norm_w.double().cpu()
    r = plain.rotate(lat[:, None, rank:], pos, freqs, "half")[:, 0]
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    got_q = q.view(T, heads, P)
    close(got_q[..., : dim + rot], q_ref, tol)
    assert float(got_q[..., dim + rot:].float().abs().sum()) == 0            # the padding of a head is zero
    close(kvrow, torch.cat([c, r], 1), tol)
    close(kc[3, 0, 1], torch.cat([c, r], 1)[5 + 65], tol)                     # token 65 of the second sequence
    close(kc[2, 0, 4], torch.cat([c, r], 1)[4], tol)
    # the small product per head, with what follows a head's inputs carried along or skipped
    w = torch.randn(heads, dim, rank, device=DEV).to(dtype)
    packed = got_q[..., : dim + rot].reshape(T, -1).contiguous()
    out = torch.empty(T, heads * (rank + rot), dtype=dtype, device=DEV)
    K.head_project(out, packed, w, heads, dim, rank, extra=rot)
    src = packed.double().cpu().view(T, heads, dim + rot)
    want = torch.cat([torch.einsum("thd,hdn->thn", src[..., :dim], w.double().cpu()), src[..., dim:]], -1)
    close(out.view(T, heads, -1), want, 1e-5 if dtype == torch.float32 else 1e-2)
    out2 = torch.empty(T, heads * rank, dtype=dtype, device=DEV)
    K.head_project(out2, q, w, heads, dim, rank, x_pitch=P)
    close(out2.view(T, heads, -1), want[..., :rank], 1e-5 if dtype == torch.float32 else 1e-2)
    # the few rows of a decode step go through a kernel of their own (eight tokens a block)
    for n in (1, 5, 13):
        few = torch.full((n, heads * (rank + rot)), float("nan"), dtype=dtype, device=DEV)
        K.head_project(few, packed[:n].contiguous(), w, heads, dim, rank, extra=rot)
        close(few.view(n, heads, -1), want[:n], 1e-5 if dtype == torch.float32 else 1e-2)
        few2 = torch.empty(n, heads * rank, dtype=dtype, device=DEV)
        K.head_project(few2, q[:n].contiguous(), w, heads, dim, rank, x_pitch=P)
        close(few2.view(n, heads, -1), want[:n, :, :rank], 1e-5 if dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------- attention

def plain_attention(q, k, v, scale, mask, sinks=None, gate=None):
    """q [T, nq, dk], k [T, nkv, dk], v [T, nkv, dv] of one sequence -> [T, nq, dv]."""
    T, nq, _ = q.shape
    nkv = k.shape[1]
    out = torch.zeros(T, nq, v.shape[-1], dtype=F64)
    for h in range(nq):
        g = h // (nq // nkv)
        p = plain.softmax_rows((q[:, h] @ k[:, g].T) * scale, mask, sink=None if sinks is None else sinks[h])
        out[:, h] = p @ v[:, g]
        if gate is not None:
            out[:, h] *= plain.sigmoid(gate[:, h:h + 1])
    return out


def ring_cache(k, v, ring, dtype, values_in_keys=False):
    """One sequence's rows as the cache holds them once all are stored: row j at j % ring of pages taken in a
    scrambled order (the last writer of a ring row wins).  k [L, nkv, dk], v [L, nkv, dv]."""
    L, nkv, dk = k.shape
    rows = min(L, ring) if ring else L
    n = (rows + PAGE - 1) // PAGE
    ids = [5, 2, 7, 0, 3, 6, 1, 4][:n]
    kc = paged(8, nkv, dk, dtype)
    vc = None if values_in_keys else paged(8, nkv, v.shape[-1], dtype)
    for j in range(L):
        r = j % ring if ring else j
        kc[ids[r // PAGE], :, r % PAGE] = k[j].to(dtype)
        if vc is not None:
            vc[ids[r // PAGE], :, r % PAGE] = v[j].to(dtype)
    table = torch.full((1, 8), -1, dtype=torch.int32, device=DEV)
    table[0, :n] = torch.tensor(ids, dtype=torch.int32)
    return kv_view(kc, vc, table, ring)


CASES = [   # nq, nkv, dk, dv, size, mask, sink, gate, values in keys
    (4, 2, 12, 20, 7, "chunk", False, True, False),
    (3, 1, 26, 20, 5, "window", True, False, True),
    (6, 2, 64, 64, 70, "chunk", False, True, False),        # the tensor-core kernels in bfloat16
    (4, 4, 128, 128, 100, "chunk", True, True, False),
    (4, 1, 128, 96, 130, "window", True, False, True),      # cached rows of 128 with the values inside
    (2, 2, 64, 64, 33, "window", True, False, False),
    (2, 1, 40, 40, 1, "chunk", False, False, False),        # a token sees itself alone
    (4, 1, 320, 256, 130, "window", True, False, True),     # wide rows with the values inside: the kernel for them
    (18, 1, 576, 512, 100, "window", True, True, True),     # (more heads than a tile of 16)
    (6, 2, 48, 32, 5, "chunk", False, False, True),
]


@pytest.mark.parametrize("nq,nkv,dk,dv,size,mask,sink,gate,inside", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_of_prompts_and_single_tokens(K, nq, nkv, dk, dv, size, mask, sink, gate, inside, dtype):
    """A prompt of 150 tokens beside one of 3 through ``attn_prefill``; then every one of the positions 140 .. 149,
    decoded alone over the paged ring that holds what came before it, through ``attn_decode`` (the split kernel where
    it takes the sizes, the plain one cut into runs elsewhere)."""
    L = 150
    scale = 2.0 / math.sqrt(dk)
    q = torch.randn(L, nq, dk, dtype=F64)
    k = torch.randn(L, nkv, dk, dtype=F64)
    v = k[..., :dv].clone() if inside else torch.randn(L, nkv, dv, dtype=F64)
    sinks = torch.randn(nq, dtype=F64) * 2 if sink else None
    g = torch.randn(L, nq, dtype=F64) * 2 if gate else None
    m = plain.chunk_mask(L, size) if mask == "chunk" else plain.window_mask(L, size)
    want = plain_attention(q, k, v, scale, m, sinks, g)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    dev = lambda t: None if t is None else t.to(device=DEV, dtype=torch.float32)
    # ---- the prompt, with a short one behind it
    lens = [L, 3]
    batch = step_batch(lens)
    T = L + 3
    pad = lambda t: torch.cat([t, t[:3]], 0)
    qd, kd, vd = (pad(t).reshape(T, -1).to(device=DEV, dtype=dtype) for t in (q, k, v))
    out = torch.empty(T, nq * dv, dtype=dtype, device=DEV)
    gd = None if g is None else dev(pad(g)).contiguous()
    K.attn_prefill(out, qd, kd, vd, batch, nq, nkv, dk, scale, 0.0, size, dv=dv, mask=mask, sinks=dev(sinks), gate=gd)
    close(out[:L].view(L, nq, dv), want, tol)
    close(out[L:].view(3, nq, dv), plain_attention(q[:3], k[:3], v[:3], scale, m[:3, :3], sinks, None if g is None else g[:3]), tol)
    # ---- single tokens over the ring
    ring = (size + PAGE - 1) // PAGE * PAGE
    for pos in range(140, 150):
        kv = ring_cache(k[: pos + 1], v[: pos + 1], ring, dtype, values_in_keys=inside)
        b = step_batch([1], decode_from=[pos])
        wide = inside and K.attn_decode_fast(dtype, dk, 1)
        o = torch.empty(1, nq * (dk if wide else dv), dtype=dtype, device=DEV)
        gd = None if g is None else dev(g[pos: pos + 1]).contiguous()
        K.attn_decode(o, q[pos: pos + 1].reshape(1, -1).to(device=DEV, dtype=dtype), kv, b, nq, nkv, dk, scale, 0.0, size,
                      dv=dv, mask=mask, sinks=dev(sinks), gate=gd)
        close(o.view(1, nq, -1)[..., :dv], want[pos: pos + 1], tol)
    # the plain kernel cut into several runs gives what it gives in one
    kv = ring_cache(k, v, ring, dtype, values_in_keys=inside)
    b = step_batch([1], decode_from=[L - 1])
    outs = []
    for n in (1, 3):
        o = torch.empty(1, nq * dv, dtype=dtype, device=DEV)
        K.attn_decode_plain(o, q[L - 1: L].reshape(1, -1).to(device=DEV, dtype=dtype), kv.k, kv.v, kv.page_table, b.slots,
                            b.len_after, nq, nkv, dk, scale, 0.0, size, ring, dv=dv, mask=mask, sinks=dev(sinks),
                            gate=None if g is None else dev(g[L - 1: L]).contiguous(), n_splits=n)
        outs.append(o)
        close(o.view(1, nq, dv), want[L - 1: L], tol)


@pytest.mark.parametrize("mask,size", [("window", 75), ("chunk", 75), ("window", 130), ("chunk", 64), ("window", 190), ("chunk", 128)])
@pytest.mark.parametrize("dk", [40, 128])
def test_a_key_at_the_edge_shows(K, mask, size, dk):
    """One key's score stands far above all others.  Placed at the first position that the last token still sees,
    the output is that key's value; placed one position earlier it must not matter at all.  Prompts and single tokens,
    plain kernels (32-bit) and tensor-core kernels (bfloat16 with a head size they take)."""
    L, nq, nkv = 200, 2, 1
    last = L - 1
    first_seen = last - last % size if mask == "chunk" else last - size + 1
    for dtype in (torch.float32, torch.bfloat16):
        for at, seen in ((first_seen, True), (first_seen - 1, False)):
            q = torch.randn(L, nq, dk, dtype=F64) * 0.1
            k = torch.randn(L, nkv, dk, dtype=F64) * 0.1
            v = torch.randn(L, nkv, dk, dtype=F64)
            k[at] = q[last, 0] * 400.0                      # head 0 of the last token scores about 4 dk there
            k[last] = -q[last, 0] * 400.0                   # (and lowest on itself)
            ring = (size + PAGE - 1) // PAGE * PAGE
            batch = step_batch([L])
            out = torch.empty(L, nq * dk, dtype=dtype, device=DEV)
            to = lambda t: t.reshape(t.shape[0], -1).to(device=DEV, dtype=dtype)
            K.attn_prefill(out, to(q), to(k), to(v), batch, nq, nkv, dk, 1.0, 0.0, size, mask=mask)
            o = torch.empty(1, nq * dk, dtype=dtype, device=DEV)
            K.attn_decode(o, to(q[last:]), ring_cache(k, v, ring, dtype), step_batch([1], decode_from=[last]), nq, nkv, dk,
                          1.0, 0.0, size, mask=mask)
            for got in (out[last, :dk], o[0, :dk]):
                d = float((got.double().cpu() - v[at, 0]).abs().max())
                assert (d < 0.05) == seen, (dtype, at, seen, d)
