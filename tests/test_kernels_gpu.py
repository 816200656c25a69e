"""Each CUDA kernel alone against a plain float32 statement of the same operation, at sizes the
tiny models do not have (rows that are no multiple of 8, head sizes 16 to 256, groups of 1, 3
and 8, vocabularies that are no power of two), in float32 and bfloat16."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as pq

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def ops():
    from litellmengine_b200.csrc import ops as o
    return o


def status():
    return torch.zeros(2, dtype=torch.int32, device=DEV)


def close(a, b, tol):
    a, b = a.double().cpu(), b.double().cpu()
    scale = max(1.0, float(b.abs().max()))
    err = float((a - b).abs().max())
    assert err <= tol * scale, f"max error {err:.3e} > {tol * scale:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden", [100, 64, 4104])
def test_embedding(dtype, hidden):
    torch.manual_seed(0)
    table = torch.randn(331, hidden).to(DT[dtype])
    ids = torch.tensor([0, 330, 7, 7, 123], dtype=torch.int32)
    st = status()
    out = ops().embedding(ids.to(DEV), table.to(DEV), st)
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table.float()[ids.long()])
    assert st.tolist() == [0, 0]
    bad = torch.tensor([3, 331, 5, -1], dtype=torch.int32)
    out = ops().embedding(bad.to(DEV), table.to(DEV), st).cpu()
    code, where = st.tolist()
    assert code == 1 and where in (1, 3)                 # recorded, not trapped
    assert out[1].abs().sum() == 0 and out[3].abs().sum() == 0 and torch.equal(out[0], table.float()[3])


@pytest.mark.parametrize("xd,dd,od", [("float32", None, "float32"), ("float32", "bfloat16", "bfloat16"),
                                      ("float32", "float32", "bfloat16"), ("bfloat16", "bfloat16", "float32")])
@pytest.mark.parametrize("hidden", [100, 48, 5120])
def test_rmsnorm_with_residual_add_and_row_pick(xd, dd, od, hidden):
    torch.manual_seed(1)
    x = torch.randn(37, hidden).to(DT[xd])
    delta = (torch.randn(37, hidden) * 0.5).to(DT[dd]) if dd else None
    w = 1 + 0.1 * torch.randn(hidden)
    eps = 3e-5
    v = x.float() + (delta.float() if delta is not None else 0)
    ref = pq.rms_norm(v, w, eps)
    tol = 1e-6 if od == "float32" else 4e-3
    xg = x.to(DEV)
    out = ops().rmsnorm(xg, w.to(DEV), eps, DT[od], delta=delta.to(DEV) if delta is not None else None,
                        write_sum=delta is not None)
    close(out, ref, tol)
    if delta is not None:                                 # the sum went back into x
        close(xg, v, 1e-6 if xd == "float32" else 4e-3)
    rows = torch.tensor([36, 0, 5, 5], dtype=torch.int32)
    out = ops().rmsnorm(x.to(DEV), w.to(DEV), eps, DT[od], delta=delta.to(DEV) if delta is not None else None,
                        rows=rows.to(DEV))
    close(out, ref[rows.long()], tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("inter", [100, 24, 3000])
def test_silu_and_mul(dtype, inter):
    torch.manual_seed(2)
    gu = (torch.randn(19, 2 * inter) * 3).to(DT[dtype])
    ref = pq.silu_and_mul(gu.float()[:, :inter], gu.float()[:, inter:])
    close(ops().silu_and_mul(gu.to(DEV)), ref, 1e-6 if dtype == "float32" else 8e-3)


def test_residual_add_and_scatter():
    h = torch.randn(7, 33)
    d = torch.randn(7, 33).to(torch.bfloat16)
    hg = h.to(DEV)
    ops().residual_add(hg, d.to(DEV))
    assert torch.equal(hg.cpu(), h + d.float())
    dst = torch.zeros(4, 5, dtype=torch.int32, device=DEV)
    st = status()
    idx = torch.tensor([0, 19, 7, 99, 3], dtype=torch.int32, device=DEV)
    val = torch.tensor([11, 12, 13, 14, 15], dtype=torch.int32, device=DEV)
    ops().scatter_int32(dst, idx, val, torch.tensor([4], dtype=torch.int32, device=DEV), 5, st)
    flat = dst.flatten().tolist()
    assert flat[0] == 11 and flat[19] == 12 and flat[7] == 13 and flat[3] == 0      # count 4: the fifth is not applied
    assert st.tolist()[0] == 2                            # index 99 is outside: recorded and skipped


def build_cache(k, v, page, table, num_pages, dtype):
    """k, v [T, nkv, d] of ONE request laid into pages by `table` (logical -> physical)."""
    T, nkv, d = k.shape
    cache = torch.zeros(num_pages, 2, nkv, page, d)
    cache += 77.0                                          # stale data everywhere: reads must be bounded
    for t in range(T):
        cache[table[t // page], 0, :, t % page] = k[t]
        cache[table[t // page], 1, :, t % page] = v[t]
    return cache.to(DT[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,page,rot,T", [(4, 4, 16, 4, 16, 29), (6, 2, 48, 16, 48, 29), (8, 1, 128, 8, 64, 29),
                                                 (3, 3, 256, 32, 256, 29), (2, 1, 80, 16, 40, 29),
                                                 # head sizes 64 and 128 rotated whole: the register kernel, with
                                                 # one head per warp (few tokens) and four (11 heads: a ragged group)
                                                 (5, 3, 128, 16, 128, 29), (5, 3, 128, 16, 128, 93),
                                                 (7, 2, 64, 8, 64, 29), (7, 2, 64, 8, 64, 93)])
def test_qk_norm_rope_kv_write(dtype, nq, nkv, d, page, rot, T):
    torch.manual_seed(3)
    theta, eps = 50000.0, 1e-5
    heads = nq + 2 * nkv
    qkv = torch.randn(T, heads * d)
    qw, kw = 1 + 0.2 * torch.randn(d), 1 + 0.2 * torch.randn(d)
    # two requests: slot 2 holds positions 5.., slot 0 holds positions 40..
    first = T - 12
    pos = torch.cat([torch.arange(5, 5 + first), torch.arange(40, 40 + 12)]).to(torch.int32)
    entry = torch.cat([torch.zeros(first), torch.ones(12)]).to(torch.int32)
    slots = torch.tensor([2, 0], dtype=torch.int32)
    width = (max(52, 5 + first) + page - 1) // page + 1
    num_pages = 2 * width + 5
    table = torch.full((3, width), -1, dtype=torch.int32)
    perm = torch.randperm(num_pages)[:2 * width].to(torch.int32)
    table[2], table[0] = perm[:width], perm[width:]
    cache = torch.zeros(num_pages, 2, nkv, page, d, dtype=DT[dtype], device=DEV)
    i = torch.arange(rot // 2, dtype=torch.float32)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float32).double(), (-(2.0 * i) / float(rot)).double()).float()
    st = status()
    q = ops().qk_norm_rope_kv_write(qkv.to(DEV), cache, pos.to(DEV), entry.to(DEV), slots.to(DEV), table.to(DEV),
                                    qw.to(DEV), kw.to(DEV), eps, inv.to(DEV), rot, nq, nkv, d, page, True, st,
                                    q_dtype=DT[dtype])
    assert st.tolist() == [0, 0]
    x = qkv.view(T, heads, d)

    def rope_part(t):                                      # rotate the first `rot` dims, pass the rest
        r = pq.rope(t[..., :rot].contiguous(), pos, theta) if rot == d else \
            torch.cat([_rope_custom(t[..., :rot], pos, inv), t[..., rot:]], dim=-1)
        return r
    qr = rope_part(pq.rms_norm(x[:, :nq], qw, eps))
    kr = rope_part(pq.rms_norm(x[:, nq:nq + nkv], kw, eps))
    vr = x[:, nq + nkv:]
    tol = 2e-6 if dtype == "float32" else 8e-3
    close(q.view(T, nq, d), qr, tol)
    c = cache.float().cpu()
    for t in range(T):
        p, s = int(pos[t]), int(slots[entry[t]])
        pg = int(table[s, p // page])
        close(c[pg, 0, :, p % page], kr[t], tol)
        close(c[pg, 1, :, p % page], vr[t], tol)
    touched = {(int(table[int(slots[entry[t]]), int(pos[t]) // page]), int(pos[t]) % page) for t in range(T)}
    for pg in range(num_pages):
        for r in range(page):
            if (pg, r) not in touched:
                assert c[pg, :, :, r].abs().sum() == 0, "a row nobody owns was written"
    # with the step's table of sines and cosines instead of its own: the same bits
    angles = ops().rope_angles(pos.to(DEV), inv.to(DEV))
    ang = pos.float()[:, None] * inv[None, :]
    close(angles[..., 0], torch.sin(ang.double()), 1e-6)
    close(angles[..., 1], torch.cos(ang.double()), 1e-6)
    cache2 = torch.zeros_like(cache)
    q2 = ops().qk_norm_rope_kv_write(qkv.to(DEV), cache2, pos.to(DEV), entry.to(DEV), slots.to(DEV), table.to(DEV),
                                     qw.to(DEV), kw.to(DEV), eps, inv.to(DEV), rot, nq, nkv, d, page, True, st,
                                     q_dtype=DT[dtype], angles=angles)
    assert torch.equal(q2, q) and torch.equal(cache2, cache)


def _rope_custom(x, pos, inv):
    half = x.shape[-1] // 2
    ang = pos.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def test_qk_write_refuses_a_bad_page_without_trapping():
    nq = nkv = 1
    d, page = 16, 4
    cache = torch.zeros(2, 2, nkv, page, d, device=DEV)
    table = torch.tensor([[0, 9]], dtype=torch.int32, device=DEV)      # page 9 does not exist
    st = status()
    z = lambda *a: torch.tensor(a, dtype=torch.int32, device=DEV)
    ops().qk_norm_rope_kv_write(torch.randn(2, 3 * d, device=DEV), cache, z(3, 4), z(0, 0), z(0), table, None, None,
                                0.0, None, 0, nq, nkv, d, page, True, st)
    assert st.tolist() == [3, 1] and cache[1].abs().sum() == 0


def attention_case(dtype, nq, nkv, d, page, lens, window=None, spike=None, q_rows=None, seed=0):
    """Requests of the given lengths in shuffled pages; queries at `q_rows` (default: all
    positions).  `spike` = (request, key position): that key is made to dominate its row, so a
    wrong page or row shows as a different value vector, not as a small shift of a mean."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    width = max((n + page - 1) // page for n in lens)
    num_pages = B * width + 3
    perm = torch.randperm(num_pages, generator=g).to(torch.int32)
    table = torch.full((B, width), -1, dtype=torch.int32)
    caches, qs, refs, pos_l, ent_l = [], [], [], [], []
    cache = torch.zeros(num_pages, 2, nkv, page, d) + 55.0
    for b, n in enumerate(lens):
        table[b, :width] = perm[b * width:(b + 1) * width]
        q = torch.randn(n, nq, d, generator=g)
        k = torch.randn(n, nkv, d, generator=g)
        v = torch.randn(n, nkv, d, generator=g)
        if spike is not None and spike[0] == b:
            j = spike[1]
            k[j] = 0.0
            k[j, :, 0] = 6.0
            q[:, :, 0] = 6.0 * math.sqrt(d) / 6.0 * 3.0          # score of key j: 18, far above the rest
            v[j] = torch.arange(d, dtype=torch.float32)[None, :] + 100.0
        rows = list(range(n)) if q_rows is None else [r for r in q_rows[b]]
        for t in range(n):
            cache[table[b, t // page], 0, :, t % page] = k[t]
            cache[table[b, t // page], 1, :, t % page] = v[t]
        kk, vv = (k.to(DT[dtype]).float(), v.to(DT[dtype]).float())
        qq = q.to(DT[dtype]).float()
        full = pq.causal_attention(qq.double(), kk.double(), vv.double(), window=window)
        qs.append(qq[rows])
        refs.append(full[rows])
        pos_l += rows
        ent_l += [b] * len(rows)
    q_all = torch.cat(qs).reshape(-1, nq * d).to(DT[dtype])
    out = ops().paged_attention_generic(
        q_all.to(DEV), cache.to(DT[dtype]).to(DEV), torch.tensor(pos_l, dtype=torch.int32, device=DEV),
        torch.tensor(ent_l, dtype=torch.int32, device=DEV), torch.arange(B, dtype=torch.int32, device=DEV),
        table.to(DEV), nq, nkv, d, page, window, 1.0 / math.sqrt(d), status())
    return out.view(-1, nq, d), torch.cat(refs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,page", [(4, 4, 16, 4), (6, 2, 48, 16), (8, 1, 128, 16), (3, 3, 256, 8),
                                           (5, 5, 80, 64), (16, 2, 64, 1)])
def test_paged_attention_sizes(dtype, nq, nkv, d, page):
    out, ref = attention_case(dtype, nq, nkv, d, page, lens=[1, 37, 130])
    close(out, ref, 3e-6 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", [0, 15, 16, 17, 31, 32, 255, 256, 300, 479])
def test_a_far_key_among_hundreds_is_found(dtype, key):
    """One key dominates; its value vector is unmistakable.  Keys at page edges (page 16),
    at tile edges (32), the first and the last."""
    n = 480
    out, ref = attention_case(dtype, 6, 2, 32, 16, lens=[40, n], spike=(1, key),
                              q_rows=[[39], [n - 1, max(key, 1)]], seed=key)
    close(out, ref, 3e-6 if dtype == "float32" else 1e-2)
    assert float(out[1].float().mean()) > 90.0           # the spiked value really carried the row


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 16, 17, 33, 200])
def test_window_edges(dtype, window):
    """The key just inside the window counts, the one just outside does not: spike each."""
    n = 230
    for inside in (True, False):
        qpos = n - 1
        key = qpos - window + 1 if inside else qpos - window
        if key < 0:
            continue
        out, ref = attention_case(dtype, 4, 2, 32, 16, lens=[n], window=window, spike=(0, key),
                                  q_rows=[[qpos, window // 2]], seed=window)
        close(out, ref, 3e-6 if dtype == "float32" else 1e-2)
        assert (float(out[0].float().mean()) > 90.0) == inside


def test_attention_refuses_sizes_it_was_not_written_for():
    from litellmengine_b200.csrc.ops import KernelError
    z = lambda *a: torch.tensor(a, dtype=torch.int32, device=DEV)
    for nq, nkv, d in ((4, 3, 32), (2, 1, 24), (2, 1, 272)):
        with pytest.raises(KernelError, match="refused"):
            ops().paged_attention_generic(torch.zeros(1, nq * d, device=DEV), torch.zeros(1, 2, nkv, 4, d, device=DEV),
                                          z(0), z(0), z(0), z(0).view(1, 1), nq, nkv, d, 4, None, 1.0, status())
    with pytest.raises(KernelError, match="CUDA device"):
        ops().silu_and_mul(torch.zeros(2, 8))


@pytest.mark.parametrize("vocab", [331, 1000, 151936])
def test_argmax_rows_ties_go_low(vocab):
    torch.manual_seed(5)
    lg = torch.randn(6, vocab)
    lg[1, 17] = lg[1, vocab - 1] = 9.0                    # tie: lowest index wins
    lg[2, :] = 0.5
    lg[3, vocab - 1] = 12.0
    got = ops().argmax_rows(lg.to(DEV)).tolist()
    assert got == [pq.argmax_token(r) for r in lg] and got[1] == 17 and got[2] == 0 and got[3] == vocab - 1


@pytest.mark.parametrize("vocab", [331, 50021])
def test_sample_rows_follow_their_own_streams(vocab):
    from litellmengine_b200.sampling import slot_state_row
    torch.manual_seed(6)
    lg = torch.randn(5, vocab) * 2
    temps = [0.8, 0.0, 1.5, 0.8, 0.3]
    seeds = [11, 12, 13, 11, 2**40 + 5]
    state = torch.tensor([slot_state_row(s, 0, t) for s, t in zip(seeds, temps)] + [[0, 0, 0, 0]] * 3, dtype=torch.int32)
    row_slot = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32)
    sd = state.to(DEV)
    draws = []
    for step in range(6):
        tok = ops().sample_rows(lg.to(DEV), row_slot.to(DEV), sd).tolist()
        draws.append(tok)
        for r, t in enumerate(tok):
            if temps[r] == 0.0:
                assert t == pq.argmax_token(lg[r])
                continue
            u = ops().sampler_uniform(seeds[r], step)
            p = pq.temperature_probs(lg[r], temps[r]).double()
            cdf = torch.cumsum(p, 0)
            lo = float(cdf[t - 1]) if t > 0 else 0.0
            assert lo - 1e-5 <= u <= float(cdf[t]) + 1e-5, f"row {r} step {step}: u={u} not in token {t}'s interval"
    assert sd[:, 2].tolist()[:5] == [6, 0, 6, 6, 6]       # sampled rows advanced their counters
    assert len({tuple(d) for d in draws}) > 1             # the stream moves
    # same logits and same seed give the same draws: rows 0 and 3
    lg2 = lg.clone()
    lg2[3] = lg2[0]
    sd = state.to(DEV)
    for _ in range(4):
        tok = ops().sample_rows(lg2.to(DEV), row_slot.to(DEV), sd).tolist()
        assert tok[0] == tok[3]
    us = [ops().sampler_uniform(7, c) for c in range(2000)]
    assert 0.0 <= min(us) and max(us) < 1.0 and abs(np.mean(us) - 0.5) < 0.03


# ---- the tuned bfloat16 attention kernels ------------------------------------------------------
def fast_case(kernel, nq, nkv, d, page, reqs, window=None, spike=None, splits=1, seed=0, ramp=None):
    """reqs: [(keys in the cache after the step, queries at the end)].  Runs `kernel` ('decode' or
    'prefill') over all queries and returns (out, reference) for the query rows."""
    g = torch.Generator().manual_seed(seed)
    B = len(reqs)
    width = max((n + page - 1) // page for n, _ in reqs) + 1
    num_pages = B * width + 2
    perm = torch.randperm(num_pages, generator=g).to(torch.int32)
    table = torch.full((B, width), -1, dtype=torch.int32)
    cache = torch.zeros(num_pages, 2, nkv, page, d) + 33.0
    qs, refs, pos_l, ent_l, q_start, q_len, kv_len, tiles, dec_rows = [], [], [], [], [], [], [], [], []
    row = 0
    for b, (n, nqr) in enumerate(reqs):
        table[b] = perm[b * width:(b + 1) * width]
        q = torch.randn(n, nq, d, generator=g)
        k = torch.randn(n, nkv, d, generator=g)
        v = torch.randn(n, nkv, d, generator=g)
        if spike is not None and spike[0] == b:
            j = spike[1]
            k[j] = 0.0
            k[j, :, 0] = 6.0
            q[:, :, 0] = 3.0 * math.sqrt(d)
            v[j] = torch.arange(d, dtype=torch.float32)[None, :] + 100.0
        if ramp is not None and ramp[0] == b:                # scores that climb with the key index, by ramp[1] in all
            k[:, :, 0] = torch.linspace(0.0, ramp[1], n)[:, None]
            q[:, :, 0] = math.sqrt(d)
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
        for t in range(n):
            cache[table[b, t // page], 0, :, t % page] = k[t]
            cache[table[b, t // page], 1, :, t % page] = v[t]
        full = pq.causal_attention(q.double(), k.double(), v.double(), window=window)
        qs.append(q[n - nqr:])
        refs.append(full[n - nqr:])
        pos_l += list(range(n - nqr, n))
        ent_l += [b] * nqr
        q_start.append(row)
        q_len.append(nqr)
        kv_len.append(n)
        if nqr == 1:
            dec_rows.append(row)
        for q0 in range(0, nqr, ops().PREFILL_TILE_ROWS):
            tiles += [b, q0]
        row += nqr
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    q_all = torch.cat(qs).reshape(-1, nq * d).to(torch.bfloat16).to(DEV)
    out = torch.zeros_like(q_all)
    st = status()
    cache = cache.to(torch.bfloat16).to(DEV)
    scale = 1.0 / math.sqrt(d)
    if kernel == "decode":
        rows = None if len(dec_rows) == row else i32(dec_rows)
        ops().paged_attention_decode(q_all, out, cache, rows, len(dec_rows), i32(pos_l), i32(ent_l),
                                     i32(list(range(B))), table.to(DEV), nq, nkv, d, page, window, scale, splits, st)
    else:
        fn = ops().paged_attention_prefill_tcgen05 if kernel == "prefill_tcgen05" else ops().paged_attention_prefill
        fn(q_all, out, cache, i32(tiles).view(-1, 2), len(tiles) // 2, i32(list(range(B))),
           i32(q_start), i32(q_len), i32(kv_len), table.to(DEV), nq, nkv, d, page, window, scale, st)
    assert st.tolist() == [0, 0]
    return out.view(-1, nq, d), torch.cat(refs)


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (6, 6, 64, 16), (7, 1, 64, 8), (16, 2, 128, 64),
                                           (6, 2, 128, 4), (5, 1, 64, 16)])
def test_decode_attention_kernel(nq, nkv, d, page, splits):
    out, ref = fast_case("decode", nq, nkv, d, page, [(1, 1), (37, 1), (300, 1), (513, 1), (64, 1)], splits=splits)
    close(out, ref, 1e-2)


@pytest.mark.parametrize("key", [0, 15, 16, 31, 32, 127, 128, 255, 256, 511, 600, 639])
def test_decode_kernel_finds_a_far_key(key):
    out, ref = fast_case("decode", 8, 2, 128, 16, [(50, 1), (640, 1)], spike=(1, key), splits=5, seed=key)
    close(out, ref, 1e-2)
    assert float(out[1].float().mean()) > 90.0


@pytest.mark.parametrize("window", [1, 16, 33, 200])
def test_decode_kernel_window_edges(window):
    n = 300
    for inside in (True, False):
        key = n - 1 - window + 1 if inside else n - 1 - window
        out, ref = fast_case("decode", 4, 2, 64, 16, [(n, 1)], window=window, spike=(0, key), splits=3, seed=window)
        close(out, ref, 1e-2)
        assert (float(out[0].float().mean()) > 90.0) == inside


def test_decode_kernel_on_a_subset_of_rows():
    """A mixed batch: only the single-token entries go to the decode kernel; other rows of the
    output are left alone."""
    out, ref = fast_case("decode", 8, 2, 128, 16, [(40, 7), (99, 1), (64, 3), (130, 1)], splits=2)
    rows = [7, 11]
    close(out[rows], ref[rows], 1e-2)
    rest = [i for i in range(12) if i not in rows]
    assert out[rest].abs().sum() == 0


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (6, 6, 64, 16), (3, 1, 64, 8), (4, 2, 128, 64), (6, 2, 128, 4)])
def test_prefill_attention_kernel(nq, nkv, d, page):
    reqs = [(2, 2), (64, 64), (65, 65), (130, 130), (200, 7), (333, 129), (128, 64), (70, 2)]
    out, ref = fast_case("prefill", nq, nkv, d, page, reqs)
    close(out, ref, 1e-2)


@pytest.mark.parametrize("key", [0, 15, 16, 63, 64, 65, 127, 128, 300, 383, 384, 400, 449])
def test_prefill_kernel_finds_a_far_key(key):
    """The portion is the last 66 positions of 450; the spiked key lies before it, at its first
    position, inside it, at tile and page edges.  Queries before the key must not see it."""
    n, nqr = 450, 66
    out, ref = fast_case("prefill", 4, 2, 128, 16, [(30, 30), (n, nqr)], spike=(1, key), seed=key)
    close(out, ref, 1e-2)
    first_q = n - nqr
    means = out[30:].float().mean(dim=(1, 2))
    for i in range(nqr):
        assert (float(means[i]) > 90.0) == (first_q + i >= key)


@pytest.mark.parametrize("window", [1, 5, 64, 65, 100])
def test_prefill_kernel_window_edges(window):
    n, nqr = 300, 150
    for inside in (True, False):
        qpos = n - 1
        key = qpos - window + 1 if inside else qpos - window
        out, ref = fast_case("prefill", 4, 2, 64, 16, [(n, nqr)], window=window, spike=(0, key), seed=window)
        close(out, ref, 1e-2)
        assert (float(out[-1].float().mean()) > 90.0) == inside


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 16, 512), (8, 100, 520), (3, 331, 80), (16, 48, 4096), (9, 1000, 1544),
                                   (5, 17, 8), (8, 6144, 4096), (17, 331, 80), (24, 1000, 1544), (32, 4096, 1024),
                                   (29, 1024, 3072)])
def test_skinny_product(M, N, K, out_dtype):
    """The weight-streaming product for decode steps, its weights fetched box by box from their plain
    layout, against float64, at sizes that are no multiple of its tiles (N of 64, K of 256, M of 8, 16
    or 32: the 32-token tile is what small products take for 17 to 32 rows)."""
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    got = ops().linear_skinny(x.to(DEV), w.to(DEV), DT[out_dtype])
    assert got.dtype == DT[out_dtype] and got.shape == (M, N)
    close(got, ref, 2e-5 if out_dtype == "float32" else 6e-3)
    assert ops().stream_status(DEV).tolist() == [0, 0]
    lib = torch.mm(x.to(DEV), w.to(DEV).t(), out_dtype=torch.float32)
    close(got, lib, 2e-5 if out_dtype == "float32" else 6e-3)      # and against the library product


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 16, 512), (8, 100, 520), (3, 331, 80), (7, 48, 4096), (8, 1000, 1544),
                                   (5, 17, 8), (8, 6144, 4096), (2, 4096, 12288),
                                   (9, 100, 520), (16, 331, 80), (13, 1000, 1544), (16, 6144, 4096), (11, 4096, 12288),
                                   (12, 70, 384), (16, 64, 128), (17, 100, 520), (32, 1000, 1544), (25, 6144, 1024)])
def test_skinny_product_over_tiled_weights(M, N, K, out_dtype):
    """The same product reading a copy of the weights stored tile by tile (one bulk copy per
    stage): same sums as over the plain layout, at sizes with ragged edge tiles."""
    torch.manual_seed(M * 1000 + N + 1)
    x = torch.randn(M, K).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16).to(DEV)
    ref = x.double().cpu() @ w.double().cpu().T
    plain = ops().linear_skinny(x, w, DT[out_dtype])
    ops().prepare_streaming(w)
    assert w.data_ptr() in ops()._tiled
    got = ops().linear_skinny(x, w, DT[out_dtype])
    close(got, ref, 2e-5 if out_dtype == "float32" else 6e-3)
    assert torch.equal(got, plain)                          # same order of additions: bit for bit
    parts = ops().linear_skinny(x, w, DT[out_dtype], partials_ok=True)
    close(ops().as_tensor(parts), ref, 2e-5 if out_dtype == "float32" else 6e-3)
    assert ops().stream_status(DEV).tolist() == [0, 0]
    key = w.data_ptr()
    del w, got, plain, parts
    import gc
    gc.collect()
    assert key not in ops()._tiled                          # the copy went with its weight


@pytest.mark.parametrize("M", [1, 8, 13])
def test_output_head_at_the_real_vocabulary(M):
    """151,936 x 4,096 weights (1.2 GB, past 2^29 elements) through the streaming product, plain and
    tiled: against the library's product in float32 accumulation, and the argmax of its rows."""
    torch.manual_seed(M)
    x = torch.randn(M, 4096, device=DEV).to(torch.bfloat16)
    w = (torch.randn(151936, 4096, device=DEV) * 0.02).to(torch.bfloat16)
    w[151935] = x[0] * 0.05                                  # the last row wins for the first token
    lib = torch.mm(x, w.t(), out_dtype=torch.float32)
    plain = ops().linear_skinny(x, w, torch.float32)
    close(plain, lib, 2e-5)
    ops().prepare_streaming(w)
    assert w.data_ptr() in ops()._tiled
    tiled = ops().linear_skinny(x, w, torch.float32)
    assert torch.equal(tiled, plain)
    assert ops().argmax_rows(tiled).tolist() == torch.argmax(lib, dim=1).tolist()
    assert int(ops().argmax_rows(tiled)[0]) == 151935
    assert ops().stream_status(DEV).tolist() == [0, 0]


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,N,K", [(256, 256, 64), (128, 64, 512), (300, 520, 136), (513, 1000, 1544), (17, 8, 8),
                                   (1100, 776, 448), (2048, 1024, 4096), (260, 6144, 640), (2048, 2560, 128),
                                   (512, 9472, 64), (4000, 2552, 200)])
def test_paired_tcgen05_product(T, N, K, out_dtype):
    """The product that two CTAs of a cluster compute together (256 tokens x 256 features a tile)
    against float64, at sizes that are no multiple of its tiles; with fewer tiles than clusters (taken
    whole or in halves), exactly one round of whole tiles, and whole rounds followed by halves (both
    accumulators, the ring of stages wrapping, units of 256 and 128 columns in one launch)."""
    torch.manual_seed(T * 1000 + N)
    x = torch.randn(T, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    got = ops().linear_pair(x.to(DEV), w.to(DEV), DT[out_dtype])
    assert got.dtype == DT[out_dtype] and got.shape == (T, N)
    close(got, ref, 2e-5 if out_dtype == "float32" else 6e-3)
    if out_dtype == "float32":                              # added onto a float32 tensor in place
        base = torch.randn(T, N)
        acc = ops().linear_pair(x.to(DEV), w.to(DEV), torch.float32, out=base.to(DEV), accumulate=True)
        assert torch.equal(acc, base.to(DEV) + got)
    assert ops().stream_status(DEV).tolist() == [0, 0]


@pytest.mark.parametrize("T,inter,K", [(256, 128, 64), (300, 264, 136), (700, 1000, 520), (130, 8, 64), (2048, 3072, 1024),
                                       (2048, 1280, 128), (520, 4736, 64)])
def test_paired_tcgen05_gate_up_product(T, inter, K):
    """The same with silu(gate) * up in its epilogue: bit for bit what the bfloat16 product followed
    by the separate activation kernel gives when both add in the same order; checked here against
    float64 products rounded to bfloat16 before the activation."""
    torch.manual_seed(T + inter)
    x = torch.randn(T, K).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K) * 0.05).to(torch.bfloat16)
    gu = (x.double() @ w.double().T).to(torch.bfloat16).double()
    ref = (gu[:, :inter] / (1.0 + torch.exp(-gu[:, :inter]))) * gu[:, inter:]
    got = ops().linear_pair_silu_mul(x.to(DEV), w.to(DEV))
    assert got.dtype == torch.bfloat16 and got.shape == (T, inter)
    close(got, ref, 1e-2)           # a product that lands on a bfloat16 rounding boundary may fall either way
    two_step = ops().silu_and_mul(ops().linear_pair(x.to(DEV), w.to(DEV), torch.bfloat16))
    assert torch.equal(got, two_step)
    assert ops().stream_status(DEV).tolist() == [0, 0]


# ---- the tcgen05 / TMEM / TMA prompt-portion attention kernel ------------------------------------
@pytest.mark.parametrize("nq,nkv,page", [(8, 2, 16), (4, 4, 64), (3, 1, 8), (6, 2, 64), (4, 2, 32), (5, 5, 16)])
def test_prefill_tcgen05_kernel(nq, nkv, page):
    reqs = [(2, 2), (64, 64), (129, 129), (130, 3), (200, 7), (333, 129), (400, 400), (128, 128), (257, 130)]
    out, ref = fast_case("prefill_tcgen05", nq, nkv, 128, page, reqs)
    close(out, ref, 1e-2)


@pytest.mark.parametrize("key", [0, 15, 16, 127, 128, 129, 255, 256, 300, 383, 384, 400, 449])
def test_prefill_tcgen05_finds_a_far_key(key):
    n, nqr = 450, 66
    out, ref = fast_case("prefill_tcgen05", 4, 2, 128, 16, [(30, 30), (n, nqr)], spike=(1, key), seed=key)
    close(out, ref, 1e-2)
    first_q = n - nqr
    means = out[30:].float().mean(dim=(1, 2))
    for i in range(nqr):
        assert (float(means[i]) > 90.0) == (first_q + i >= key)


def test_long_contexts_decode_and_prompt_kernels():
    """Thousands of keys: block tables of hundreds of pages, sixteen key splits of twenty tiles each
    in the decode kernel, twenty-four 128-key tiles and a ring that wraps twelve times in the
    one-pass prompt kernel; a spiked key early in the context must still be found."""
    out, ref = fast_case("decode", 4, 2, 128, 16, [(5000, 1), (4097, 1)], splits=16, spike=(0, 77), seed=5)
    close(out, ref, 1e-2)
    assert float(out[0].float().mean()) > 90.0
    out, ref = fast_case("prefill_tcgen05", 4, 2, 128, 16, [(3000, 260)], spike=(0, 131), seed=6)
    close(out, ref, 1e-2)
    assert float(out[-1].float().mean()) > 90.0


@pytest.mark.parametrize("climb", [3.0, 12.0, 40.0, 150.0])
def test_prefill_tcgen05_scores_that_keep_climbing(climb):
    """The one-pass kernel keeps a reference maximum that trails the running one and rescales its
    accumulator only when the maximum has run away: scores that rise with the key index by
    `climb` over 1,500 keys (12 tiles) make that happen never, sometimes, or at every tile."""
    out, ref = fast_case("prefill_tcgen05", 4, 2, 128, 16, [(40, 40), (1500, 300)], ramp=(1, climb), seed=3)
    close(out, ref, 1e-2)


@pytest.mark.parametrize("window", [1, 5, 128, 129, 200])
def test_prefill_tcgen05_window_edges(window):
    n, nqr = 300, 150
    for inside in (True, False):
        qpos = n - 1
        key = qpos - window + 1 if inside else qpos - window
        out, ref = fast_case("prefill_tcgen05", 4, 2, 128, 16, [(n, nqr)], window=window, spike=(0, key), seed=window)
        close(out, ref, 1e-2)
        assert (float(out[-1].float().mean()) > 90.0) == inside
