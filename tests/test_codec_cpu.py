"""Property tests of the CPU codecs (the executable payload specification)."""
import math
import struct

import pytest
import torch

import hipress_b200 as hp
from hipress_b200 import ops


def gauss(n, std=0.01, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


# ----------------------------------------------------------------------------- LCG
def test_lcg_matches_recurrence():
    seed = 12345
    x = seed
    x = (1103515245 * x + 12345) % 2**32  # discarded draw
    draws = hp._C.lcg_draws(seed, 5)
    for raw_mod, unit in draws:
        x = (1103515245 * x + 12345) % 2**32
        assert raw_mod == x % 0x7FFFFFFF
        expect = struct.unpack("f", struct.pack("f", x / 4294967295.0))[0]
        assert unit == expect
        assert 0.0 <= unit <= 1.0


def test_lcg_unit_draw_multiply_equals_division():
    # the codecs convert raw draws with a double multiply; the reference divides.  Equal for all
    # 2^32 raw values (exhaustive check done offline); here: a strided sweep plus both ends.
    C = hp._C
    assert C.lcg_unit_mismatches(0, 1 << 24, 251) == 0
    assert C.lcg_unit_mismatches(0, 1 << 16, 1) == 0
    assert C.lcg_unit_mismatches((1 << 32) - (1 << 16), 1 << 16, 1) == 0
    assert C.lcg_unit_mismatches((1 << 31) - (1 << 15), 1 << 16, 1) == 0


# ----------------------------------------------------------------------------- TBQ
def test_tbq_hand_vector():
    # g[i] = (i-5)*0.004, t = 0.01, N = 10 -> bytes 40 55 5a (hand-derived from tbq_body.h:70-87)
    g = torch.tensor([(i - 5) * 0.004 for i in range(10)])
    r = torch.zeros(10)
    out = ops.tbq_compress(g, r, 0.01)
    assert out.tolist() == [0x40, 0x55, 0x5A]


@pytest.mark.parametrize("n", [1, 3, 4, 5, 17, 1000, 4099])
def test_tbq_roundtrip_and_conservation(n):
    t = 0.01
    g = gauss(n)
    r0 = gauss(n, 0.005, seed=1)
    r = r0.clone()
    payload = ops.tbq_compress(g, r, t)
    assert payload.numel() == (n + 3) // 4
    dec = torch.empty(n)
    ops.tbq_decompress(payload, dec, t)
    assert set(torch.unique(dec).tolist()) <= {-t, 0.0, t} | {float(torch.tensor(-t)), float(torch.tensor(t))}
    # what was sent plus what stayed behind equals what came in
    torch.testing.assert_close(dec + r, g + r0, atol=1e-6, rtol=0)
    # unused fields of the last byte decode to zero
    if n % 4:
        last = payload[-1].item()
        for k in range(n % 4, 4):
            assert (last >> (2 * k)) & 3 == 1


def test_tbq_inclusive_threshold():
    t = 0.5
    g = torch.tensor([0.5, -0.5, 0.49999, -0.49999])
    r = torch.zeros(4)
    payload = ops.tbq_compress(g, r, t)
    fields = [(payload[0].item() >> (2 * k)) & 3 for k in range(4)]
    assert fields == [2, 0, 1, 1]
    assert r[0] == 0 and r[1] == 0


def test_tbq_multi_payload_accumulate():
    n, t = 1001, 0.02
    payloads = []
    for s in range(3):
        payloads.append(ops.tbq_compress(gauss(n, 0.03, seed=s), torch.zeros(n), t))
    one_pass = torch.empty(n)
    ops.tbq_decompress(payloads, one_pass, t)
    seq = torch.zeros(n)
    ops.tbq_decompress(payloads[0], seq, t, add=False)
    ops.tbq_decompress(payloads[1], seq, t, add=True)
    ops.tbq_decompress(payloads[2], seq, t, add=True)
    assert torch.equal(one_pass, seq)


# ----------------------------------------------------------------------------- TernGrad
@pytest.mark.parametrize("bw", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [1, 3, 8, 9, 1000, 4099])
def test_terngrad_header_and_error_bound(bw, n):
    g = gauss(n, seed=bw + n)
    payload = ops.terngrad_compress(g, bw, enable_random=False)
    dpb = 8 // bw
    assert payload.numel() == 10 + (n + dpb - 1) // dpb
    raw = bytes(payload.tolist())
    assert raw[0] == bw
    assert raw[1] == (0 if n % dpb == 0 else dpb - n % dpb)
    mn, mx = struct.unpack("<ff", raw[2:10])
    assert mn == g.min().item() and mx == g.max().item()
    dec = torch.empty(n)
    ops.terngrad_decompress(payload, dec)
    gap = (mx - mn) / (2**bw - 1)
    # the 1e-8 in 1/(gap+1e-8) shifts level q by up to q*1e-8
    assert (dec - g).abs().max().item() <= gap / 2 + 2**bw * 1e-8 + 1e-6


@pytest.mark.parametrize("bw", [2, 4])
def test_terngrad_stochastic_is_seeded_and_unbiased(bw):
    n = 1 << 16
    g = gauss(n, seed=7)
    a = ops.terngrad_compress(g, bw, True, seed=1)
    b = ops.terngrad_compress(g, bw, True, seed=1)
    c = ops.terngrad_compress(g, bw, True, seed=2)
    assert torch.equal(a, b)
    assert not torch.equal(a, c)
    dec = torch.empty(n)
    ops.terngrad_decompress(a, dec)
    gap = (g.max() - g.min()).item() / (2**bw - 1)
    assert (dec - g).abs().max().item() <= gap + 1e-6
    assert abs((dec - g).mean().item()) < gap * 0.02


def test_terngrad_tail_byte_is_deterministic():
    n = 4 * 100 + 3
    g = gauss(n, seed=3)
    a = ops.terngrad_compress(g, 2, True, seed=11)
    b = ops.terngrad_compress(g, 2, True, seed=99)
    det = ops.terngrad_compress(g, 2, False)
    assert a[-1] == b[-1] == det[-1]


def test_terngrad_all_zero_and_constant():
    for val in (0.0, 0.25):
        g = torch.full((37,), val)
        p = ops.terngrad_compress(g, 2, False)
        dec = torch.empty(37)
        ops.terngrad_decompress(p, dec)
        assert torch.equal(dec, g)


def test_terngrad_error_feedback_conserves():
    n = 5000
    g = gauss(n, seed=5)
    r0 = gauss(n, 0.002, seed=6)
    r = r0.clone()
    p = ops.terngrad_compress(g, 2, True, seed=3, residual=r)
    dec = torch.empty(n)
    ops.terngrad_decompress(p, dec)
    torch.testing.assert_close(dec + r, g + r0, atol=2e-7, rtol=0)


def test_terngrad_rejects_bad_bitwidth_and_size():
    g = gauss(16)
    with pytest.raises(RuntimeError):
        ops.terngrad_compress(g, 3)
    with pytest.raises(RuntimeError):
        ops.terngrad_compress(g, 2, out=torch.empty(5, dtype=torch.uint8))


# ----------------------------------------------------------------------------- sparse
def _parse_sparse(payload):
    raw = bytes(payload.tolist())
    total = struct.unpack("<i", raw[:4])[0]
    k = (total - 4) // 8
    idx = list(struct.unpack(f"<{k}i", raw[4:4 + 4 * k]))
    val = list(struct.unpack(f"<{k}f", raw[4 + 4 * k:4 + 8 * k]))
    return total, idx, val


@pytest.mark.parametrize("n,keep", [(1000, 0.01), (100000, 0.001), (4097, 0.05)])
def test_graddrop_layout_and_residual(n, keep):
    g = gauss(n, seed=1)
    r0 = gauss(n, 0.003, seed=2)
    r = r0.clone()
    payload = ops.graddrop_compress(g, r, sample_rate=0.05, drop_ratio=1 - keep, seed=42)
    total, idx, val = _parse_sparse(payload)
    k = len(idx)
    # same double arithmetic as the codec: ceil(N * (1 - drop_ratio))
    expected = math.ceil(n * (1 - (1 - keep)))
    assert payload.numel() == 4 + 8 * expected
    assert 0 <= k <= expected
    assert idx == sorted(idx) and len(set(idx)) == k
    acc = g + r0
    for i, v in zip(idx, val):
        assert v == acc[i].item()
        assert r[i] == 0
    mask = torch.ones(n, dtype=torch.bool)
    mask[idx] = False
    assert torch.equal(r[mask], acc[mask])
    # every kept magnitude is at least as large as every dropped one when trimmed to k == expected
    if k == expected and k > 0:
        assert min(abs(v) for v in val) >= acc[mask].abs().max().item()
    dec = torch.zeros(n)
    ops.sparse_decompress(payload[:total], dec)
    torch.testing.assert_close(dec + r, acc, atol=0, rtol=0)


def test_sparse_overselect_trims_to_exact_topk():
    n, keep = 10000, 0.01
    v = gauss(n, seed=9)
    ref = v.clone()
    # sample_rate 0 -> threshold 0 -> everything qualifies -> must trim to the exact top-k
    payload = ops.dgc_compress(v, sample_rate=0.0, keep_fraction=keep, seed=1)
    _, idx, val = _parse_sparse(payload)
    k = math.ceil(n * keep)
    assert len(idx) == k
    top = torch.topk(ref.abs(), k).indices.sort().values.tolist()
    assert idx == top
    assert all(v[i] == 0 for i in idx)


def test_sparse_ties_prefer_lower_index():
    v = torch.tensor([1.0, -1.0, 1.0, 0.5, 1.0, -1.0, 0.25, 1.0])
    payload = ops.dgc_compress(v.clone(), sample_rate=0.0, keep_fraction=3 / 8, seed=0)
    _, idx, _ = _parse_sparse(payload)
    assert idx == [0, 1, 2]


def test_sparse_decompress_add_and_bounds():
    n = 100
    v = gauss(n, seed=4)
    p = ops.dgc_compress(v.clone(), 0.0, 0.1, seed=0)
    out = torch.ones(n)
    ops.sparse_decompress(p, out, add=True)
    _, idx, val = _parse_sparse(p)
    for i, x in zip(idx, val):
        assert out[i] == 1.0 + torch.tensor(x)
    bad = p.clone()
    bad[0:4] = torch.tensor(list(struct.pack("<i", 4 + 8 * 1000)), dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        ops.sparse_decompress(bad, torch.zeros(n))


# ----------------------------------------------------------------------------- ECQ
@pytest.mark.parametrize("bw", [2, 4, 8])
@pytest.mark.parametrize("n", [5, 1000, 4099])
def test_ecq_header_roundtrip_and_history(bw, n):
    g = gauss(n, seed=bw)
    h0 = gauss(n, 0.002, seed=n)
    h = h0.clone()
    alpha, beta = 1.0, 0.9
    p = ops.ecq_compress(g, h, alpha, beta, bw, seed=5)
    dpb = 8 // bw
    M = (n + dpb - 1) // dpb
    raw = bytes(p.tolist())
    total, mx = struct.unpack("<if", raw[:8])
    assert total == 10 + M and raw[8] == bw and raw[9] == M * dpb - n
    v = g + alpha * h0
    assert mx == pytest.approx(v.abs().max().item(), rel=1e-6)
    dec = torch.empty(n)
    ops.ecq_decompress(p, dec)
    gap = mx / (2 ** (bw - 1) - 1)
    assert (dec - v).abs().max().item() <= gap + 1e-6
    torch.testing.assert_close(h, beta * h0 + (v - dec), atol=1e-6, rtol=0)


def test_ecq_zero_tensor():
    g = torch.zeros(33)
    h = torch.zeros(33)
    p = ops.ecq_compress(g, h, 1.0, 1.0, 2, seed=0)
    dec = torch.ones(33)
    ops.ecq_decompress(p, dec)
    assert torch.equal(dec, torch.zeros(33))


# ----------------------------------------------------------------------------- PowerSGD
def test_powersgd_cpu_matches_fp64():
    torch.manual_seed(0)
    n, m, r = 96, 200, 4
    N = n * m - 7
    grad = torch.randn(N)
    resid = torch.randn(N) * 0.1
    Q = torch.randn(m, r)
    M = torch.zeros(n, m)
    P = torch.zeros(n, r)
    ops.powersgd_encode1(grad, resid, Q, M, P)
    M64 = torch.zeros(n * m, dtype=torch.float64)
    M64[:N] = (grad + resid).double()
    M64 = M64.view(n, m)
    torch.testing.assert_close(P.double(), M64 @ Q.double(), atol=1e-4, rtol=1e-4)
    ops.powersgd_encode2(P, M, Q)
    eye = P.double().T @ P.double()
    torch.testing.assert_close(eye, torch.eye(r, dtype=torch.float64), atol=1e-5, rtol=0)
    torch.testing.assert_close(Q.double(), M64.T @ P.double(), atol=1e-4, rtol=1e-4)
    g2, r2 = grad.clone(), torch.zeros(N)
    ops.powersgd_decode(P, Q, M, r2, g2)
    approx = (P.double() @ Q.double().T).view(-1)[:N]
    torch.testing.assert_close(g2.double(), approx, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(r2.double(), grad.double() - approx, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("n", [1 << 18, (1 << 20) + 3, 3 * (1 << 18) + 5])
def test_threaded_cpu_codecs_are_bit_identical(n):
    """TBQ and TernGrad (every bitwidth, stochastic and deterministic, with and without error feedback) on several
    threads give the bytes, residuals and decodes of the one-thread loops."""
    g = torch.randn(n, generator=torch.Generator().manual_seed(n)) * 0.01
    def run():
        out = []
        r = torch.zeros(n)
        p = ops.tbq_compress(g, r, 0.004)
        d = torch.full((n,), 0.5)
        ops.tbq_decompress([p, p], d, 0.004, add=True)
        out += [p, r, d]
        for bw in (1, 2, 4, 8):
            for rnd in (False, True):
                r = torch.zeros(n)
                p = ops.terngrad_compress(g, bw, rnd, seed=7, residual=r)
                d = torch.empty(n)
                ops.terngrad_decompress([p], d)
                out += [p, r, d]
        return out
    try:
        ops.set_cpu_threads(1)
        ref = run()
        ops.set_cpu_threads(5)
        assert ops.get_cpu_threads() == 5
        got = run()
    finally:
        ops.set_cpu_threads(1)
    assert len(ref) == len(got)
    for a, b in zip(ref, got):
        assert torch.equal(a, b)


@pytest.mark.parametrize("case", ["signed_zeros", "nan_in_the_middle", "infinities", "nan_first"])
def test_threaded_minmax_follows_element_order(case):
    """The threaded min/max scan reports the first minimum and the last maximum of the one-thread scan (visible
    for +-0.0 extremes) and takes the one-thread path whenever the tensor holds a NaN."""
    n = 1 << 19
    g = torch.zeros(n)
    if case == "signed_zeros":
        g[::3] = -0.0
        g[5::7] = 0.0
    else:
        g = torch.randn(n, generator=torch.Generator().manual_seed(3)) * 0.01
        if case == "nan_in_the_middle":
            g[n // 2 + 17] = float("nan")
        elif case == "nan_first":
            g[0] = float("nan")
        else:
            g[1000], g[n - 5] = float("inf"), float("-inf")
    try:
        ops.set_cpu_threads(1)
        ref = ops.terngrad_compress(g, 2, False, seed=1)
        ops.set_cpu_threads(6)
        got = ops.terngrad_compress(g, 2, False, seed=1)
    finally:
        ops.set_cpu_threads(1)
    assert torch.equal(ref, got)
