"""Each CUDA kernel alone against its plain statement (tests/reference_kernels.py), at sizes other
than the tiny models': widths and vocabularies that are no power of two, head sizes in steps of 16,
odd group sizes, and inputs made so that a fault in an index shows (one key that stands out among
hundreds, the window's edge, the slot of the cache)."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from reference_kernels import ReferenceKernels
from cima_b200.cache.kv import LayerKV

pytestmark = pytest.mark.gpu

REF = ReferenceKernels(compute=torch.float64)
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# one rounding to the output dtype of values of magnitude about 1, plus summation error
TOL = {"float32": 2e-5, "bfloat16": 1.6e-2}


@pytest.fixture(scope="module")
def K():
    from cima_b200.kernels import Kernels
    return Kernels(verbose=False)


def g(*shape, dtype=torch.float32, seed=0, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


def err(a, b):
    return (a.double().cpu() - b.double().cpu()).abs().max().item()


# ---------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
def test_embed(K, wdtype):
    V, H = 777, 200
    table = g(V, H, dtype=DT[wdtype])
    ids = torch.tensor([0, 776, 5, 5, 300], dtype=torch.int32)
    x = torch.full((5, H), -7.0, device="cuda")
    K.embed(ids.cuda(), table.cuda(), x, 1.0)
    assert torch.equal(x.cpu(), table[ids.long()].float())


@pytest.mark.parametrize("odtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,eps", [(200, 3e-6), (3584, 1e-6), (1, 1e-5), (1000, 1e-2)])
def test_rmsnorm(K, odtype, H, eps):
    x, w = g(13, H, seed=1, scale=3.0), 1 + g(H, seed=2, scale=0.1)
    out = torch.empty(13, H, dtype=DT[odtype], device="cuda")
    K.rmsnorm(x.cuda(), w.cuda(), eps, out)
    want = torch.empty(13, H, dtype=torch.float64)
    REF.rmsnorm(x, w, eps, want)
    assert err(out, want) <= TOL[odtype] * 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_and_residual_and_gather(K, dtype):
    T, I = 37, 328
    gu = g(T, 2 * I, dtype=DT[dtype], seed=3, scale=2.0)
    out = torch.empty(T, I, dtype=DT[dtype], device="cuda")
    for code in (0, 1, 2, 3):                           # the gate's activation: SiLU, GELU (tanh, erf), ReLU
        K.swiglu(gu.cuda(), out, code)
        want = torch.empty(T, I, dtype=torch.float64)
        REF.swiglu(gu, want, code)
        assert err(out, want) <= TOL[dtype] * 4, code
    x, d = g(T, I, seed=4), g(T, I, dtype=DT[dtype], seed=5)
    xg = x.cuda()
    K.add_residual(xg, d.cuda())
    assert torch.equal(xg.cpu(), x + d.float())
    rows = torch.tensor([36, 0, 0, 17], dtype=torch.int32)
    picked = torch.empty(4, I, device="cuda")
    K.gather_rows(xg, rows.cuda(), picked)
    assert torch.equal(picked.cpu(), xg.cpu()[rows.long()])


# ---------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M,N,K_", [(1, 192, 448), (7, 1000, 333), (130, 65, 17), (64, 64, 64)])
@pytest.mark.parametrize("combo", [("float32", "float32", "float32"), ("bfloat16", "float32", "bfloat16"),
                                   ("bfloat16", "bfloat16", "float32")])
def test_linear_plain(K, M, N, K_, combo):
    a, w, b = g(M, K_, dtype=DT[combo[0]], seed=1), g(N, K_, dtype=DT[combo[1]], seed=2, scale=0.1), g(N, seed=3)
    # guard columns around the output prove that nothing is written outside it
    # (the reference's sentinel check, src/selftest.rs:803, :837-850)
    out = torch.full((M, N), -777.0, dtype=DT[combo[2]], device="cuda")
    K.linear_plain(a.cuda(), w.cuda(), b.cuda(), out)
    want = a.double() @ w.double().t() + b.double()
    assert err(out, want) <= TOL[combo[2]] * max(1.0, want.abs().max().item())
    if combo[2] == "float32":
        acc = torch.ones(M, N, device="cuda")
        K.linear_plain(a.cuda(), w.cuda(), None, acc, accumulate=True)
        assert err(acc, 1 + a.double() @ w.double().t()) <= 2e-5 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("rows", [1, 5, 8])
@pytest.mark.parametrize("N,K_", [(300, 200), (65, 7), (1000, 3584)])
def test_linear_plain_rows_are_independent(K, rows, N, K_):
    """The same bits for a row whether it comes among 70 (the tiled kernel) or among at most 8 (the kernel of
    the decode steps, one thread per output feature): both add the products of an output in ascending k."""
    a, w, b = g(70, K_, seed=1), g(N, K_, seed=2), g(N, seed=3)
    full = torch.empty(70, N, device="cuda")
    K.linear_plain(a.cuda(), w.cuda(), b.cuda(), full)
    few = torch.empty(rows, N, device="cuda")
    K.linear_plain(a[33:33 + rows].contiguous().cuda(), w.cuda(), b.cuda(), few)
    assert torch.equal(full[33:33 + rows], few)
    acc_full, acc_few = torch.ones(70, N, device="cuda"), torch.ones(rows, N, device="cuda")
    K.linear_plain(a.cuda(), w.cuda(), None, acc_full, accumulate=True)
    K.linear_plain(a[33:33 + rows].contiguous().cuda(), w.cuda(), None, acc_few, accumulate=True)
    assert torch.equal(acc_full[33:33 + rows], acc_few)


@pytest.mark.parametrize("M", [1, 3, 7, 8])
@pytest.mark.parametrize("N,K_", [(200, 328), (1000, 192), (4608, 3584), (17, 8)])
def test_linear_skinny_modes(K, M, N, K_):
    from cima_b200.kernels import SK_ACCUM, SK_STORE, SK_STORE_F32, SK_SWIGLU
    a = g(M, K_, dtype=torch.bfloat16, seed=M)
    w = g(N, K_, dtype=torch.bfloat16, seed=N, scale=1.0 / math.sqrt(K_))
    b = g(N, seed=7)
    want = a.double() @ w.double().t()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.linear_skinny(a.cuda(), w.cuda(), b.cuda(), out, SK_STORE)
    assert err(out, want + b.double()) <= TOL["bfloat16"] * 4
    out32 = torch.empty(M, N, device="cuda")
    K.linear_skinny(a.cuda(), w.cuda(), None, out32, SK_STORE_F32)
    assert err(out32, want) <= 1e-4
    x = g(M, N, seed=9)
    xg = x.cuda()
    K.linear_skinny(a.cuda(), w.cuda(), None, xg, SK_ACCUM)
    assert err(xg, x.double() + want) <= 1e-4
    if N % 2 == 0:
        I = N // 2
        gg, uu = want[:, :I], want[:, I:]
        for code in (0, 1, 2, 3):                       # the gate's activation: SiLU, GELU (tanh, erf), ReLU
            act = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
            K.linear_skinny(a.cuda(), w.cuda(), None, act, SK_SWIGLU, act=code)
            assert err(act, REF.gate_act(gg, code) * uu) <= TOL["bfloat16"] * 4, code
        with pytest.raises(Exception, match="activation code"):
            K.linear_skinny(a.cuda(), w.cuda(), None, act, SK_SWIGLU, act=9)


def test_linear_skinny_row_does_not_depend_on_batch(K):
    from cima_b200.kernels import SK_STORE_F32
    a, w = g(8, 448, dtype=torch.bfloat16, seed=1), g(1000, 448, dtype=torch.bfloat16, seed=2)
    full = torch.empty(8, 1000, device="cuda")
    K.linear_skinny(a.cuda(), w.cuda(), None, full, SK_STORE_F32)
    for m in (1, 2, 5, 7):
        part = torch.empty(m, 1000, device="cuda")
        K.linear_skinny(a[:m].contiguous().cuda(), w.cuda(), None, part, SK_STORE_F32)
        assert torch.equal(part, full[:m])


def test_linear_skinny_refuses(K):
    from cima_b200.kernels import KernelError, SK_STORE
    a, w = g(9, 64, dtype=torch.bfloat16).cuda(), g(32, 64, dtype=torch.bfloat16).cuda()
    with pytest.raises(KernelError, match="at most 8"):
        K.linear_skinny(a, w, None, torch.empty(9, 32, dtype=torch.bfloat16, device="cuda"), SK_STORE)
    a, w = g(2, 12, dtype=torch.bfloat16).cuda(), g(32, 12, dtype=torch.bfloat16).cuda()
    with pytest.raises(KernelError, match="multiples of 8"):
        K.linear_skinny(a, w, None, torch.empty(2, 32, dtype=torch.bfloat16, device="cuda"), SK_STORE)


# ---------------------------------------------------------------------------- cache and attention
def make_kv(n_pages, nkv, page, hd, n_slots, width, ring, window, dtype, tables):
    """A layer's pages (filled with a large stale value) and block table, on the GPU and mirrored on the CPU."""
    storage = torch.full((n_pages, 2, nkv, page, hd), 50.0, dtype=dtype)
    table = torch.zeros(n_slots, width, dtype=torch.int32)
    for slot, pages in tables.items():
        table[slot, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
    cpu = LayerKV(storage, table, page, ring, window, 0)
    gpu = LayerKV(storage.cuda(), table.cuda(), page, ring, window, 0)
    return cpu, gpu


def batch_of(seqs, device):
    """seqs: list of (slot, start_pos, n_tokens) -> the arrays the kernels take."""
    row_pos, row_seq, first = [], [], [0]
    for i, (slot, start, n) in enumerate(seqs):
        row_pos += list(range(start, start + n))
        row_seq += [i] * n
        first.append(first[-1] + n)
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    tiles = sorted(((i, r0) for i, s in enumerate(seqs) for r0 in range(0, s[2], 64)), key=lambda x: -x[1])
    tc = [x for x in tiles if x[1] % 128 == 0]
    tiles.sort(key=lambda x: -(seqs[x[0]][1] + x[1]))
    return SimpleNamespace(n_q_tiles=len(tiles) if any(s[2] > 1 for s in seqs) else 0,
                           n_q_tiles_tc=len(tc), q_tile_tc_seq=t([x[0] for x in tc]), q_tile_tc_row0=t([x[1] for x in tc]),
                           q_tile_seq=t([x[0] for x in tiles]), q_tile_row0=t([x[1] for x in tiles]),
                           row_pos=t(row_pos), row_seq=t(row_seq), seq_slot=t([s[0] for s in seqs]),
                           seq_first_row=t(first), seq_len=t([s[1] + s[2] for s in seqs]),
                           n_rows=len(row_pos), n_seqs=len(seqs), prefill=all(s[1] == 0 for s in seqs),
                           max_len=max(s[1] + s[2] for s in seqs), max_rows=max(s[2] for s in seqs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(6, 2, 48, 48), (7, 7, 16, 16), (4, 1, 128, 64), (2, 2, 256, 256)])
def test_rope_append(K, dtype, nh, nkv, hd, rot):
    page = 16
    seqs = [(2, 0, 21), (0, 37, 1), (3, 5, 9)]
    tables = {2: [4, 1], 0: [7, 3, 9], 3: [0]}
    cpu, gpu = make_kv(10, nkv, page, hd, 4, 3, 0, 0, DT[dtype], tables)
    T = sum(s[2] for s in seqs)
    qkv = g(T, (nh + 2 * nkv) * hd, dtype=DT[dtype], seed=hd)
    inv = torch.pow(torch.tensor(12345.0, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).float()
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = qkv.clone()
    REF.rope_append(want, inv, rot, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_len, cpu, nh, nkv, hd)
    got = qkv.cuda()
    K.rope_append(got, inv.cuda(), rot, bg.row_pos, bg.row_seq, bg.seq_slot, bg.seq_len, gpu, nh, nkv, hd)
    assert err(got, want) <= TOL[dtype]
    assert err(gpu.storage, cpu.storage) <= TOL[dtype]
    # pages of no sequence keep their stale contents
    for p in (2, 5, 6, 8):
        assert torch.all(gpu.storage[p].float() == 50.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rope_append_long_prompt_wraps_a_ring(K, dtype):
    """A prompt longer than a windowed group's ring: every place must end up with its newest
    position, whichever block of the launch ran last."""
    nh, nkv, hd, page, window = 2, 2, 32, 16, 20
    ring = -(-window // page) + 1                      # 3 pages = 48 positions
    seqs = [(1, 0, 200), (0, 0, 30), (2, 0, 49)]
    tables = {1: [5, 0, 7], 0: [3, 8, 1], 2: [2, 4, 6]}
    cpu, gpu = make_kv(9, nkv, page, hd, 3, ring, ring, window, DT[dtype], tables)
    T = sum(s[2] for s in seqs)
    qkv = g(T, (nh + 2 * nkv) * hd, dtype=DT[dtype], seed=11)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float()
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = qkv.clone()
    REF.rope_append(want, inv, hd, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_len, cpu, nh, nkv, hd)
    for _ in range(3):
        got = qkv.cuda()
        gpu.storage.fill_(50.0)
        K.rope_append(got, inv.cuda(), hd, bg.row_pos, bg.row_seq, bg.seq_slot, bg.seq_len, gpu, nh, nkv, hd)
        assert err(gpu.storage, cpu.storage) <= TOL[dtype]
    # position 199 of the long prompt is where the ring says, holding the rotated key of row 199
    e, off = (199 // page) % ring, 199 % page
    assert err(gpu.storage[tables[1][e], 0, :, off], want[199].view(-1, hd)[nh:nh + nkv]) <= TOL[dtype]


def test_rope_is_a_rotation_by_position_times_frequency(K):
    """Independent check: pair (i, i + d/2) as a complex number is multiplied by exp(i * p * f_i)."""
    nh, nkv, hd, theta = 2, 1, 32, 10000.0
    T = 5
    qkv = g(T, (nh + 2 * nkv) * hd, seed=1)
    pos = torch.tensor([0, 1, 17, 255, 4000], dtype=torch.int32)
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    got = qkv.cuda()
    z = torch.zeros(T, dtype=torch.int32, device="cuda")
    K.rope_append(got, inv.float().cuda(), hd, pos.cuda(), z, z[:1], z[:1], None, nh, nkv, hd)
    u = qkv.double().view(T, nh + 2 * nkv, hd)[:, :nh + nkv]
    c = torch.complex(u[..., :hd // 2], u[..., hd // 2:]) * torch.polar(torch.ones(T, hd // 2, dtype=torch.float64),
                                                                        pos.double()[:, None] * inv[None])[:, None, :]
    want = torch.cat([c.real, c.imag], dim=-1)
    gotq = got.cpu().double().view(T, nh + 2 * nkv, hd)
    assert (gotq[:, :nh + nkv] - want).abs().max().item() <= 3e-3 * 1e-2 + 4000 * 1.2e-7 * 4   # angle rounding at p = 4000
    assert torch.equal(gotq[:, nh + nkv:], qkv.double().view(T, -1, hd)[:, nh + nkv:])           # v untouched


def fill_cache(cpu, gpu, slot, k, v):
    """Write keys/values [n, nkv, hd] of positions 0..n-1 into a slot's pages (ring aware)."""
    for j in range(k.shape[0]):
        e = j // cpu.page_size
        if cpu.ring_pages:
            e %= cpu.ring_pages
        page = int(cpu.block_table[slot, e])
        cpu.storage[page, 0, :, j % cpu.page_size] = k[j]
        cpu.storage[page, 1, :, j % cpu.page_size] = v[j]
    gpu.storage.copy_(cpu.storage)


def scattered_tables(lens, slots, page, ring=0, seed=0):
    """Pages for each slot, drawn from a shuffled pool; returns (tables, pool size, table width)."""
    need = [min(-(-n // page), ring) if ring else -(-n // page) for n in lens]
    total = sum(need) + 3
    order = np.random.default_rng(seed).permutation(total).tolist()
    tables, k = {}, 0
    for slot, n in zip(slots, need):
        tables[slot] = order[k:k + n]
        k += n
    return tables, total, max(need)


@pytest.mark.parametrize("nh,nkv,hd", [(28, 4, 128), (14, 2, 64)])
def test_attention_decode_with_many_live_splits(K, nh, nkv, hd):
    """One sequence of 5,000 positions (79 pages) beside a short one: 33, 40 and 64 splits that all have pages (the
    short sequence's blocks beyond its pages have none), and the number the wrapper chooses for one long sequence
    alone (64), against the float64 statement; key 4,321 stands out for head 0."""
    lens, slots, page = [5000, 70], [2, 0], 64
    tables, n_pages, width = scattered_tables(lens, slots, page, seed=hd + 1)
    cpu, gpu = make_kv(n_pages, nkv, page, hd, 4, width, 0, 0, torch.bfloat16, tables)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(2, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=5)
    for i, (slot, n) in enumerate(zip(slots, lens)):
        k, v = g(n, nkv, hd, dtype=torch.bfloat16, seed=30 + i), g(n, nkv, hd, dtype=torch.bfloat16, seed=40 + i)
        if i == 0:
            k[4321, 0] = qkv[0, :hd] * 6.0
        fill_cache(cpu, gpu, slot, k, v)
    seqs = [(slots[i], lens[i] - 1, 1) for i in range(2)]
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = torch.zeros(2, nh * hd, dtype=torch.float64)
    REF.attention_plain(qkv, cpu, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_first_row, want, nh, nkv, hd, scale, 0, True)
    out = torch.empty(2, nh * hd, dtype=torch.bfloat16, device="cuda")
    for n_splits in (33, 40, 64):
        out.fill_(7.0)
        K.attention_decode(qkv.cuda(), gpu, bg.seq_slot, bg.seq_len, out, nh, nkv, hd, scale, 0, n_splits=n_splits)
        assert err(out, want) <= TOL["bfloat16"], n_splits
    from cima_b200.engine.profile import StepProfile
    K.profile = seen = StepProfile()
    try:
        out.fill_(7.0)
        K.attention_decode(qkv[:1].cuda(), gpu, bg.seq_slot[:1], bg.seq_len[:1], out[:1], nh, nkv, hd, scale, 0, max_len=5000)
    finally:
        K.profile = None
    assert [l.name for l in seen.launches] == ["attention_decode[64 splits]"]
    assert err(out[:1], want[:1]) <= TOL["bfloat16"]


@pytest.mark.parametrize("dtype,page", [("float32", 16), ("bfloat16", 16), ("bfloat16", 64)])
@pytest.mark.parametrize("nh,nkv,hd", [(6, 2, 48), (7, 1, 128), (4, 4, 16), (28, 4, 128), (3, 3, 80), (40, 2, 64), (2, 1, 112)])
def test_attention_decode_over_cache(K, dtype, page, nh, nkv, hd):
    """Three sequences of unequal length in scattered pages; a far key stands out in one of them.
    Pages of 64 in bfloat16 take the split-KV tensor-core kernel, the others the plain one."""
    lens = [300, 1, 77]
    slots = [1, 3, 0]
    tables, n_pages, width = scattered_tables(lens, slots, page, seed=hd)
    cpu, gpu = make_kv(n_pages, nkv, page, hd, 4, width, 0, 0, DT[dtype], tables)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(3, (nh + 2 * nkv) * hd, dtype=DT[dtype], seed=3)
    for i, (slot, n) in enumerate(zip(slots, lens)):
        k, v = g(n, nkv, hd, dtype=DT[dtype], seed=10 + i), g(n, nkv, hd, dtype=DT[dtype], seed=20 + i)
        if i == 0:
            # key 13 of 300 is the query of head 0 scaled up: nearly all the weight falls on it
            k[13, 0] = qkv[0, :hd] * 6.0
        fill_cache(cpu, gpu, slot, k, v)
    seqs = [(slots[i], lens[i] - 1, 1) for i in range(3)]
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = torch.zeros(3, nh * hd, dtype=torch.float64)
    REF.attention_plain(qkv, cpu, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_first_row, want, nh, nkv, hd, scale, 0, True)
    out = torch.empty(3, nh * hd, dtype=DT[dtype], device="cuda")
    K.attention(qkv.cuda(), gpu, bg, out, nh, nkv, hd, scale, 0, True)
    assert err(out, want) <= TOL[dtype]
    plain = torch.empty_like(out)
    K.attention_plain(qkv.cuda(), gpu, bg.row_pos, bg.row_seq, bg.seq_slot, bg.seq_first_row, plain, nh, nkv, hd, scale, 0, True)
    assert err(plain, want) <= TOL[dtype]
    if dtype == "bfloat16" and page == 64:
        # more splits than pages too; up to 8 merge inside a cluster, more through a second kernel; ``early``
        # fetches the first pages before the wait on the previous kernel (which here writes ``out`` only)
        for n_splits in (1, 2, 3, 5, 8, 9, 32):
            for early in (False, True):
                out.fill_(7.0)
                K.attention_decode(qkv.cuda(), gpu, bg.seq_slot, bg.seq_len, out, nh, nkv, hd, scale, 0,
                                   n_splits=n_splits, early=early)
                assert err(out, want) <= TOL[dtype], (n_splits, early)


@pytest.mark.parametrize("dtype,page", [("float32", 16), ("bfloat16", 16), ("bfloat16", 64)])
@pytest.mark.parametrize("window,n", [(40, 200), (16, 17), (33, 33), (64, 500), (100, 1000), (1, 70)])
def test_attention_decode_window_edge(K, dtype, page, window, n):
    """A ring of pages; the key just outside the window stands out and must not be seen, the one just
    inside must."""
    nh, nkv, hd = 4, 2, 32
    ring = -(-window // page) + 1
    tables, n_pages, width = scattered_tables([n], [1], page, ring=ring, seed=window)
    cpu, gpu = make_kv(n_pages, nkv, page, hd, 2, ring, ring, window, DT[dtype], tables)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(1, (nh + 2 * nkv) * hd, dtype=DT[dtype], seed=4)
    k, v = g(n, nkv, hd, dtype=DT[dtype], seed=5), g(n, nkv, hd, dtype=DT[dtype], seed=6)
    inside, outside = n - window, n - window - 1
    if outside >= 0:
        k[outside, 0] = qkv[0, :hd] * 8.0          # would take all the weight of head 0 if it were seen
    k[inside, 1] = qkv[0, 2 * hd:3 * hd] * 8.0     # head 2 reads kv head 1: must be seen
    # only what a ring still holds: the newest positions
    fill_cache(cpu, gpu, 1, k, v)
    bg = batch_of([(1, n - 1, 1)], "cuda")
    # the statement: plain softmax over the visible keys of the full, unwrapped sequence
    want = torch.zeros(1, nh * hd, dtype=torch.float64)
    for h in range(nh):
        gk = h // (nh // nkv)
        lo = max(0, n - window)
        s = (k[lo:n, gk].double() @ qkv[0, h * hd:(h + 1) * hd].double()) * scale
        want[0, h * hd:(h + 1) * hd] = torch.softmax(s, 0) @ v[lo:n, gk].double()
    out = torch.empty(1, nh * hd, dtype=DT[dtype], device="cuda")
    K.attention(qkv.cuda(), gpu, bg, out, nh, nkv, hd, scale, window, True)
    assert err(out, want) <= TOL[dtype]
    assert err(out[0, 2 * hd:3 * hd], v[inside, 1]) <= 5e-2      # head 2 is (nearly) that one value
    if dtype == "bfloat16" and page == 64:
        for n_splits in (1, 2, 7, 8, 16):
            for early in (False, True):
                out.fill_(7.0)
                K.attention_decode(qkv.cuda(), gpu, bg.seq_slot, bg.seq_len, out, nh, nkv, hd, scale, window,
                                   n_splits=n_splits, early=early)
                assert err(out, want) <= TOL[dtype], (n_splits, early)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 2, 48, 0), (7, 1, 128, 0), (4, 2, 64, 50), (2, 2, 256, 0),
                                              (28, 4, 128, 0), (5, 5, 16, 7), (4, 2, 96, 64), (2, 1, 32, 65),
                                              (3, 1, 112, 200), (2, 2, 80, 1)])
def test_attention_prefill_over_the_step(K, dtype, nh, nkv, hd, window):
    """Ragged prompts in one launch; keys and values come from the step's own rows."""
    lens = [130, 1, 67, 300]
    seqs = [(i, 0, n) for i, n in enumerate(lens)]
    T = sum(lens)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(T, (nh + 2 * nkv) * hd, dtype=DT[dtype], seed=hd + nh)
    # in the last sequence, key 5 stands out for the last query of head 0 (a far key among hundreds)
    last = T - 1
    first4 = T - 300
    qkv[first4 + 5, nh * hd:(nh + 1) * hd] = qkv[last, :hd] * 6.0
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = torch.zeros(T, nh * hd, dtype=torch.float64)
    REF.attention_plain(qkv, None, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_first_row, want, nh, nkv, hd, scale, window, False)
    out = torch.empty(T, nh * hd, dtype=DT[dtype], device="cuda")
    K.attention(qkv.cuda(), None, bg, out, nh, nkv, hd, scale, window, False)
    assert err(out, want) <= TOL[dtype]
    plain = torch.empty_like(out)
    K.attention_plain(qkv.cuda(), None, bg.row_pos, bg.row_seq, bg.seq_slot, bg.seq_first_row, plain, nh, nkv, hd, scale, window, False)
    assert err(plain, want) <= TOL[dtype]


@pytest.mark.parametrize("lens", [[130, 1, 67, 300], [128], [1], [257, 256, 255], [700, 40]])
@pytest.mark.parametrize("nh,nkv,window", [(7, 1, 0), (4, 2, 0), (28, 4, 0), (4, 2, 50), (2, 2, 200), (3, 1, 128), (2, 1, 1)])
@pytest.mark.parametrize("hd", [128, 64])
def test_attention_prefill_tcgen05(K, lens, nh, nkv, window, hd):
    """The tcgen05 attention of ragged prompts (head_dim 64 and 128) against the float64 statement: sequences that
    end inside a block of 128, a far key that stands out, windows with edges inside and between tiles."""
    seqs = [(i, 0, n) for i, n in enumerate(lens)]
    T = sum(lens)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=nh + T)
    if lens[-1] > 6 and (window == 0 or window >= lens[-1]):
        # in the last sequence, key 5 stands out for the last query of head 0 (a far key among hundreds)
        qkv[T - lens[-1] + 5, nh * hd:(nh + 1) * hd] = qkv[T - 1, :hd] * 6.0
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = torch.zeros(T, nh * hd, dtype=torch.float64)
    REF.attention_plain(qkv, None, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_first_row, want, nh, nkv, hd, scale, window, False)
    out = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attention_prefill_tc(qkv.cuda(), bg, out, nh, nkv, hd, scale, window)
    assert K.device_errors() == 0
    assert err(out, want) <= TOL["bfloat16"]


def first_launch_on_long_sequences(n_seqs=8, n=8192, nh=28, nkv=4, hd=128):
    """Run by the test below in a process of its own, where the launch is the kernel's first: then its loads are
    slow (nothing of the buffer is in any cache or translation buffer) and the roles of a block drift apart."""
    from cima_b200.kernels import Kernels
    K = Kernels(verbose=False)
    T = n_seqs * n
    gen = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    bg = batch_of([(i, 0, n) for i in range(n_seqs)], "cuda")
    out = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    K.attention_prefill_tc(qkv, bg, out, nh, nkv, hd, scale, 0)
    assert K.device_errors() == 0, "a bounded wait ran out in the kernel's first launch"
    for seq, h in ((0, 0), (n_seqs - 1, nh - 1), (n_seqs // 2, nh // 2)):     # some heads whole, in float64
        rows = slice(seq * n, (seq + 1) * n)
        kvh = h // (nh // nkv)
        q = qkv[rows, h * hd:(h + 1) * hd].double()
        k = qkv[rows, (nh + kvh) * hd:(nh + kvh + 1) * hd].double()
        v = qkv[rows, (nh + nkv + kvh) * hd:(nh + nkv + kvh + 1) * hd].double()
        sc = (q @ k.T) * scale
        sc.masked_fill_(torch.ones(n, n, dtype=torch.bool, device="cuda").triu(1), float("-inf"))
        want = torch.softmax(sc, dim=-1) @ v
        got = out[rows, h * hd:(h + 1) * hd].double()
        assert (got - want).abs().max().item() <= TOL["bfloat16"], (seq, h)
    print("first launch sound")


def test_attention_prefill_tcgen05_long_sequences_of_64_wide_heads():
    """Four sequences of 8,192 rows with 14 heads of 64 in 2 groups (128 key tiles a block at the narrow head size),
    three heads whole against float64."""
    first_launch_on_long_sequences(n_seqs=4, n=8192, nh=14, nkv=2, hd=64)


@pytest.mark.parametrize("attempt", [0, 1])
def test_attention_prefill_tcgen05_first_launch_on_long_sequences(attempt):
    """Eight sequences of 8,192 rows at the 7B head shape as the first launch of a fresh process.  With one barrier for
    the probabilities of both score buffers, the softmax warps could announce two tiles while the issuing thread
    still waited for a late tile of V, and its wait was answered a phase late: about every second fresh process ran
    into the bounded wait.  Two processes, since the drift is a matter of timing."""
    import os, subprocess, sys
    here = os.path.dirname(os.path.abspath(__file__))
    code = f"import sys; sys.path[:0] = [{here!r}, {os.path.dirname(here)!r}]; import test_kernels_gpu as t; t.first_launch_on_long_sequences()"
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "first launch sound" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("nh,nkv,hd", [(6, 2, 48), (28, 4, 128), (4, 4, 16)])
@pytest.mark.parametrize("window,ring", [(0, 0), (90, 0), (40, 2)])
def test_attention_of_sequences_that_go_on(K, nh, nkv, hd, window, ring):
    """Several query rows per sequence over the paged cache (the step's own keys are in the pages too) against the
    float64 statement: a sequence deep into its cache, one that starts, one across a page's edge, one with more than
    two blocks of rows; stale keys behind every sequence's end; a window, and a window through a ring of two pages."""
    page = 64
    seqs = [(2, 100, 64), (0, 0, 5), (3, 63, 2)] + ([] if ring else [(1, 500, 150)])
    width = ring or 11
    order = torch.randperm(4 * width, generator=torch.Generator().manual_seed(5)).tolist()
    tables = {slot: order[slot * width:(slot + 1) * width] for slot in range(4)}
    cpu, gpu = make_kv(4 * width, nkv, page, hd, 4, width, ring, window, torch.bfloat16, tables)
    cpu.storage.copy_(g(*cpu.storage.shape, dtype=torch.bfloat16, seed=hd + window))
    gpu.storage.copy_(cpu.storage)
    T = sum(s[2] for s in seqs)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=nh + T)
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = torch.zeros(T, nh * hd, dtype=torch.float64)
    REF.attention_plain(qkv, cpu, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_first_row, want, nh, nkv, hd, scale, window, True)
    out = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attention_extend(qkv.cuda(), gpu, bg, out, nh, nkv, hd, scale, window)
    assert err(out, want) <= TOL["bfloat16"]
    # the dispatcher takes the same kernel for such a batch
    out2 = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attention(qkv.cuda(), gpu, bg, out2, nh, nkv, hd, scale, window, True)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 128), (6, 1, 64)])
@pytest.mark.parametrize("window", [0, 90, 300])
def test_attention_of_sequences_that_go_on_by_many_rows_tcgen05(K, nh, nkv, hd, window):
    """The tcgen05 attention with its keys from the cache's pages (by TMA through the block table): a sequence of 260
    rows deep into its cache, one that starts, one of 130 rows; stale keys behind every end; windows."""
    page = 64
    seqs = [(2, 100, 260), (0, 0, 5), (1, 380, 130)]
    width = 9
    order = torch.randperm(4 * width, generator=torch.Generator().manual_seed(6)).tolist()
    tables = {slot: order[slot * width:(slot + 1) * width] for slot in range(4)}
    cpu, gpu = make_kv(4 * width, nkv, page, hd, 4, width, 0, window, torch.bfloat16, tables)
    cpu.storage.copy_(g(*cpu.storage.shape, dtype=torch.bfloat16, seed=hd + window + 1))
    gpu.storage.copy_(cpu.storage)
    T = sum(s[2] for s in seqs)
    scale = 1.0 / math.sqrt(hd)
    qkv = g(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, seed=nh + T)
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    want = torch.zeros(T, nh * hd, dtype=torch.float64)
    REF.attention_plain(qkv, cpu, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_first_row, want, nh, nkv, hd, scale, window, True)
    out = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attention_prefill_tc(qkv.cuda(), bg, out, nh, nkv, hd, scale, window, kv=gpu)
    assert K.device_errors() == 0
    assert err(out, want) <= TOL["bfloat16"]
    out2 = torch.full((T, nh * hd), 7.0, dtype=torch.bfloat16, device="cuda")
    K.attention(qkv.cuda(), gpu, bg, out2, nh, nkv, hd, scale, window, True)      # the dispatcher's choice for such a batch
    assert torch.equal(out, out2)


# ---------------------------------------------------------------------------- sampling
def test_argmax_ties_go_to_the_higher_index(K):
    V = 1000
    x = g(5, V, seed=1)
    x[0, 17] = x[0, 900] = 9.0
    x[1, :] = -3.0
    x[2, 999] = 50.0
    x[3, 0] = 50.0
    tok = torch.empty(5, dtype=torch.int32, device="cuda")
    K.argmax(x.cuda(), tok)
    assert tok.tolist() == [900, 999, 999, 0, int(torch.nonzero(x[4] == x[4].max()).max())]


# ---------------------------------------------------------------------------- norm folded into the skinny product
@pytest.mark.parametrize("M", [1, 5, 7, 8])
@pytest.mark.parametrize("N,K_", [(200, 328), (4608, 3584), (1000, 192)])
def test_skinny_accumulate_leaves_sums_of_squares_and_the_next_product_folds_the_norm(K, M, N, K_):
    """x += a W1^T leaves per-tile sums of squares of the updated rows; the next product takes the rows,
    the norm's weight and those sums and must equal RMSNorm followed by the product."""
    from cima_b200.kernels import SK_ACCUM, SK_STORE, SK_STORE_F32, SK_SWIGLU
    H = K_
    a = g(M, N, dtype=torch.bfloat16, seed=1)
    w1 = g(H, N, dtype=torch.bfloat16, seed=2, scale=1.0 / math.sqrt(N))
    x0 = g(M, H, seed=3)
    x = x0.cuda()
    ssq = torch.full((M, -(-H // 16)), -1.0, device="cuda")
    K.linear_skinny(a.cuda(), w1.cuda(), None, x, SK_ACCUM, ssq)
    want_x = x0.double() + a.double() @ w1.double().t()
    assert err(x, want_x) <= 1e-4
    assert err(ssq.sum(dim=1), (x.double() ** 2).sum(dim=1)) <= 1e-3 * max(1.0, float((want_x ** 2).sum(dim=1).max()))
    # the writer also leaves the rows times the next norm's weight; the product after the norm reads those
    nw = 1 + g(H, seed=4, scale=0.1)
    xb = x0.cuda()
    ssq_b = torch.full_like(ssq, -1.0)
    xw = torch.full((M, H), 9.0, dtype=torch.bfloat16, device="cuda")
    K.linear_skinny(a.cuda(), w1.cuda(), None, xb, SK_ACCUM, ssq_b, nw.cuda(), xw)
    assert torch.equal(xb, x) and torch.equal(ssq_b, ssq)
    assert torch.equal(xw, (x * nw.cuda()).to(torch.bfloat16))
    eps = 1e-5
    xd = x.double().cpu()
    h = (xd / torch.sqrt((xd * xd).mean(dim=1, keepdim=True) + eps) * nw.double())
    w2 = g(2 * 96, H, dtype=torch.bfloat16, seed=5, scale=1.0 / math.sqrt(H))
    b2 = g(2 * 96, seed=6)
    want = h @ w2.double().t()
    out = torch.empty(M, 192, dtype=torch.bfloat16, device="cuda")
    K.linear_skinny_norm(xw, ssq, eps, w2.cuda(), b2.cuda(), out, SK_STORE)
    assert err(out, want + b2.double()) <= TOL["bfloat16"] * 4
    out32 = torch.empty(M, 192, device="cuda")
    K.linear_skinny_norm(xw, ssq, eps, w2.cuda(), None, out32, SK_STORE_F32)
    # the operand is bf16(x * w): one bfloat16 rounding per term against the float64 statement
    assert err(out32, want) <= TOL["bfloat16"] * 2
    act = torch.empty(M, 96, dtype=torch.bfloat16, device="cuda")
    K.linear_skinny_norm(xw, ssq, eps, w2.cuda(), None, act, SK_SWIGLU)
    gg, uu = want[:, :96], want[:, 96:]
    assert err(act, gg / (1 + torch.exp(-gg)) * uu) <= TOL["bfloat16"] * 4


def test_embed_leaves_sums_of_squares(K):
    table = g(300, 200, dtype=torch.bfloat16)
    ids = torch.tensor([0, 299, 7], dtype=torch.int32)
    x = torch.empty(3, 200, device="cuda")
    ssq = torch.empty(3, 1, device="cuda")
    K.embed(ids.cuda(), table.cuda(), x, 1.0, ssq)
    assert err(ssq[:, 0], (table[ids.long()].double() ** 2).sum(dim=1)) <= 1e-3
    nw = (1 + g(200, seed=4, scale=0.1)).cuda()
    x2, ssq2 = torch.empty_like(x), torch.empty_like(ssq)
    xw = torch.empty(3, 200, dtype=torch.bfloat16, device="cuda")
    K.embed(ids.cuda(), table.cuda(), x2, 1.0, ssq2, nw, xw)
    assert torch.equal(x2, x) and torch.equal(ssq2, ssq)
    assert torch.equal(xw, (x * nw).to(torch.bfloat16))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(5, 200), (64, 3584), (300, 1000)])
def test_add_rmsnorm_equals_the_two_kernels(K, dtype, T, H):
    x0, d, w = g(T, H, seed=1, scale=2.0), g(T, H, dtype=DT[dtype], seed=2), 1 + g(H, seed=3, scale=0.1)
    xa, xb = x0.cuda(), x0.cuda()
    ha = torch.empty(T, H, dtype=DT[dtype], device="cuda")
    hb = torch.empty_like(ha)
    K.add_rmsnorm(xa, d.cuda(), w.cuda(), 1e-5, ha)
    K.add_residual(xb, d.cuda())
    K.rmsnorm(xb, w.cuda(), 1e-5, hb)
    assert torch.equal(xa, xb) and torch.equal(ha, hb)
    want = torch.empty(T, H, dtype=torch.float64)
    REF.rmsnorm(x0 + d.float(), w, 1e-5, want)
    assert err(ha, want) <= TOL[dtype] * 4


@pytest.mark.parametrize("M,N,K_", [(256, 256, 64), (300, 328, 200), (2048, 1000, 448), (513, 3584, 192), (130, 66, 72),
                                    (1, 8, 8), (257, 264, 72), (1000, 200, 136)])
def test_gemm_tcgen05_pair_modes(K, M, N, K_):
    """The product on pairs of SMs (cta_group::2) against float64, every epilogue, tails in every dimension (a last
    tile of rows that starts early to end with the matrix must store, and above all accumulate, its own rows only)."""
    from cima_b200.kernels import SK_ACCUM, SK_STORE, SK_STORE_F32, SK_SWIGLU
    a = g(M, K_, dtype=torch.bfloat16, seed=M)
    w = g(N, K_, dtype=torch.bfloat16, seed=N, scale=1.0 / math.sqrt(K_))
    b = g(N, seed=7)
    want = a.double() @ w.double().t()
    out32 = torch.full((M, N), -777.0, device="cuda")
    K.gemm_tc_pair(a.cuda(), w.cuda(), b.cuda(), out32, SK_STORE_F32)
    assert err(out32, want + b.double()) <= 1e-4
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    K.gemm_tc_pair(a.cuda(), w.cuda(), None, out, SK_STORE)
    assert err(out, want) <= TOL["bfloat16"] * 4
    x = g(M, N, seed=9)
    xg = x.cuda()
    K.gemm_tc_pair(a.cuda(), w.cuda(), None, xg, SK_ACCUM)
    assert err(xg, x.double() + want) <= 1e-4
    if N % 2 == 0:
        I = N // 2
        gg, uu = want[:, :I], want[:, I:]
        for code in (0, 1, 2, 3):                       # the gate's activation: SiLU, GELU (tanh, erf), ReLU
            act = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
            K.gemm_tc_pair(a.cuda(), w.cuda(), None, act, SK_SWIGLU, act=code)
            assert err(act, REF.gate_act(gg, code) * uu) <= TOL["bfloat16"] * 4, code
    assert K.device_errors() == 0


@pytest.mark.parametrize("M", [1, 5, 7, 8])
@pytest.mark.parametrize("nh,nkv,hd,H", [(6, 2, 48, 200), (28, 4, 128, 3584), (3, 1, 64, 192), (4, 4, 16, 64)])
def test_qkv_rope_skinny_equals_projection_then_rope_append(K, M, nh, nkv, hd, H):
    """The decode projection with rotation and cache append in its epilogue against the two separate steps
    (float64 statement): rotated q in the buffer, rotated k and v in the right pages, other pages untouched."""
    from cima_b200.kernels import SK_ACCUM
    page = 64
    N = (nh + 2 * nkv) * hd
    lens = [int(x) for x in np.random.default_rng(M).integers(1, 200, size=M)]
    slots = list(np.random.default_rng(M + 1).permutation(M + 3)[:M])
    tables, n_pages, width = scattered_tables(lens, slots, page, seed=hd + M)
    cpu, gpu = make_kv(n_pages, nkv, page, hd, M + 3, width, 0, 0, torch.bfloat16, tables)
    seqs = [(int(slots[i]), lens[i] - 1, 1) for i in range(M)]
    bc, bg = batch_of(seqs, "cpu"), batch_of(seqs, "cuda")
    a = g(M, H, dtype=torch.bfloat16, seed=1)
    w = g(N, H, dtype=torch.bfloat16, seed=2, scale=1.0 / math.sqrt(H))
    b = g(N, seed=3, scale=0.5)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float()
    # statement: projection in float64, rotation and append by the reference (rounded once at the end)
    want = (a.double() @ w.double().t() + b.double())
    REF.rope_append(want, inv, hd, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_len, cpu, nh, nkv, hd)
    qkv = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    K.qkv_rope(a.cuda(), w.cuda(), b.cuda(), qkv, inv.cuda(), bg.row_pos, bg.row_seq, bg.seq_slot, gpu, nh, nkv, hd)
    assert err(qkv[:, :nh * hd], want[:, :nh * hd]) <= TOL["bfloat16"] * 4
    assert err(gpu.storage, cpu.storage) <= TOL["bfloat16"] * 4
    # with the norm folded in: rows times the norm's weight and partial sums of squares, as an accumulating
    # product leaves them
    x = g(M, H, seed=4, scale=1.5).cuda()
    nw = (1 + g(H, seed=5, scale=0.1))
    ssq = torch.empty(M, -(-H // 16), device="cuda")
    xw = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    zero_w = torch.zeros(H, 8, dtype=torch.bfloat16, device="cuda")
    K.linear_skinny(torch.zeros(M, 8, dtype=torch.bfloat16, device="cuda"), zero_w, None, x, SK_ACCUM, ssq, nw.cuda(), xw)
    xd = x.double().cpu()
    hh = xd / torch.sqrt((xd * xd).mean(dim=1, keepdim=True) + 1e-6) * nw.double()
    want2 = hh @ w.double().t() + b.double()
    cpu2, gpu2 = make_kv(n_pages, nkv, page, hd, M + 3, width, 0, 0, torch.bfloat16, tables)
    REF.rope_append(want2, inv, hd, bc.row_pos, bc.row_seq, bc.seq_slot, bc.seq_len, cpu2, nh, nkv, hd)
    K.qkv_rope(xw, w.cuda(), b.cuda(), qkv, inv.cuda(), bg.row_pos, bg.row_seq, bg.seq_slot, gpu2, nh, nkv, hd,
               norm=(ssq, 1e-6))
    assert err(qkv[:, :nh * hd], want2[:, :nh * hd]) <= TOL["bfloat16"] * 4
    assert err(gpu2.storage, cpu2.storage) <= TOL["bfloat16"] * 4
