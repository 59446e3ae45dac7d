"""Bit-exactness against the reference's own CPU codec path.

When a checkout of the reference and nvcc are available, ``oracle/ref_oracle.cu``
is compiled against the reference headers (thrust::host policy, no GPU) and its
outputs are compared byte for byte with this library's CPU codec.  The golden
SHA-256 digests of the codec round-trip configuration (2^22 elements, 10 steps,
TBQ t=0.01 and TernGrad 2-bit seed 1) are committed in
``tests/golden/roundtrip_config.json`` so the check also runs where the
reference is absent.
"""
import hashlib
import json
import os
import shutil
import subprocess
import tempfile

import numpy as np
import pytest
import torch

from hipress_b200 import ops
import hipress_b200 as hp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("HIPRESS_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))  # a sibling checkout
GOLDEN = os.path.join(ROOT, "tests", "golden", "roundtrip_config.json")


@pytest.fixture(scope="module")
def oracle():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isdir(os.path.join(REF, "ZQ_CPP_LIB")) or not os.path.exists(nvcc):
        pytest.skip("reference checkout or nvcc not available")
    exe = os.path.join(tempfile.gettempdir(), "hipress_ref_oracle")
    src = os.path.join(ROOT, "oracle", "ref_oracle.cu")
    if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
        subprocess.run([nvcc, "-std=c++17", "-O2", "-Xcompiler", "-ffp-contract=off", "-w",
                        f"-I{REF}", "-o", exe, src], check=True)
    return exe


class Scratch:
    def __init__(self):
        self.dir = tempfile.mkdtemp(prefix="hipress_oracle_")

    def path(self, name):
        return os.path.join(self.dir, name)

    def put(self, name, t):
        t.numpy().tofile(self.path(name))
        return self.path(name)

    def get(self, name, dtype, count):
        return torch.from_numpy(np.fromfile(self.path(name), dtype=dtype, count=count).copy())

    def close(self):
        shutil.rmtree(self.dir, ignore_errors=True)


@pytest.fixture()
def scratch():
    s = Scratch()
    yield s
    s.close()


def gauss(n, std, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * std


def test_lcg_against_reference(oracle, scratch):
    for seed in (0, 1, 123456789, 0xFFFFFFFF):
        subprocess.run([oracle, "lcg", str(seed), "64", scratch.path("l.bin")], check=True)
        ref = np.fromfile(scratch.path("l.bin"), dtype=np.uint32).reshape(-1, 2)
        mine = hp._C.lcg_draws(seed, 64)
        for (a, fb), (raw, unit) in zip(ref, mine):
            assert int(a) == raw
            assert np.array([fb], dtype=np.uint32).view(np.float32)[0] == np.float32(unit)


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 7, 1023, 4096, 65537])
def test_tbq_against_reference(oracle, scratch, n):
    t = 0.01
    g = gauss(n, 0.01, n)
    r = gauss(n, 0.004, n + 1)
    scratch.put("g.bin", g)
    scratch.put("r.bin", r)
    subprocess.run([oracle, "tbq_c", scratch.path("g.bin"), scratch.path("r.bin"), str(n), repr(t),
                    scratch.path("o.bin")], check=True)
    ref_payload = scratch.get("o.bin", np.uint8, (n + 3) // 4)
    ref_resid = scratch.get("r.bin", np.float32, n)
    mine_r = r.clone()
    mine = ops.tbq_compress(g, mine_r, t)
    assert torch.equal(mine, ref_payload)
    assert torch.equal(mine_r, ref_resid)
    for add in (0, 1):
        d0 = gauss(n, 1.0, 5)
        scratch.put("d.bin", d0)
        subprocess.run([oracle, "tbq_d", scratch.path("o.bin"), str(n), repr(t), scratch.path("d.bin"),
                        str(add)], check=True)
        ref_dense = scratch.get("d.bin", np.float32, n)
        mine_dense = d0.clone()
        ops.tbq_decompress(mine, mine_dense, t, add=bool(add))
        assert torch.equal(mine_dense, ref_dense)


@pytest.mark.parametrize("bw", [1, 2, 4, 8])
@pytest.mark.parametrize("random", [0, 1])
@pytest.mark.parametrize("n", [1, 5, 8, 13, 4096, 65539])
def test_terngrad_against_reference(oracle, scratch, bw, random, n):
    g = gauss(n, 0.01, 31 * n + bw)
    seed = 1 + bw
    scratch.put("g.bin", g)
    subprocess.run([oracle, "tern_c", scratch.path("g.bin"), str(n), str(bw), str(random), str(seed),
                    scratch.path("o.bin")], check=True)
    size = ops.terngrad_payload_bytes(n, bw)
    ref_payload = scratch.get("o.bin", np.uint8, size)
    mine = ops.terngrad_compress(g, bw, bool(random), seed)
    assert torch.equal(mine, ref_payload)
    for add in (0, 1):
        d0 = gauss(n, 1.0, 9)
        scratch.put("d.bin", d0)
        subprocess.run([oracle, "tern_d", scratch.path("o.bin"), str(size), scratch.path("d.bin"),
                        str(n), str(add)], check=True)
        ref_dense = scratch.get("d.bin", np.float32, n)
        mine_dense = d0.clone()
        ops.terngrad_decompress(mine, mine_dense, add=bool(add))
        assert torch.equal(mine_dense, ref_dense)


def test_sparse_decode_against_reference(oracle, scratch):
    n = 5000
    v = gauss(n, 0.01, 3)
    payload = ops.dgc_compress(v.clone(), 0.05, 0.01, seed=7)
    total = int(payload[:4].view(torch.int32).item())
    scratch.put("p.bin", payload[:total])
    for add in (0, 1):
        d0 = gauss(n, 1.0, 4)
        scratch.put("d.bin", d0)
        subprocess.run([oracle, "gd_d", scratch.path("p.bin"), str(total), scratch.path("d.bin"),
                        str(n), str(add)], check=True)
        ref_dense = scratch.get("d.bin", np.float32, n)
        mine = d0.clone()
        ops.sparse_decompress(payload[:total], mine, add=bool(add))
        assert torch.equal(mine, ref_dense)


def _roundtrip_config_digests(use_oracle=None, scratch=None):
    """2^22 fp32 ~ N(0, 0.01^2) from torch seed 0 (fresh draw each step), 10 steps, residual carried."""
    n, steps = 1 << 22, 10
    torch.manual_seed(0)
    h_tbq, h_tern, h_tbq_dec, h_tern_dec = (hashlib.sha256() for _ in range(4))
    resid = torch.zeros(n)
    ref_resid = torch.zeros(n)
    for step in range(steps):
        g = torch.randn(n) * 0.01
        p = ops.tbq_compress(g, resid, 0.01)
        d = torch.empty(n)
        ops.tbq_decompress(p, d, 0.01)
        q = ops.terngrad_compress(g, 2, True, seed=1)
        e = torch.empty(n)
        ops.terngrad_decompress(q, e)
        for h, t in ((h_tbq, p), (h_tbq_dec, d), (h_tern, q), (h_tern_dec, e)):
            h.update(t.numpy().tobytes())
        if use_oracle:
            scratch.put("g.bin", g)
            scratch.put("r.bin", ref_resid)
            subprocess.run([use_oracle, "tbq_c", scratch.path("g.bin"), scratch.path("r.bin"), str(n),
                            "0.01", scratch.path("o.bin")], check=True)
            ref_resid = scratch.get("r.bin", np.float32, n)
            assert torch.equal(p, scratch.get("o.bin", np.uint8, n // 4)), f"tbq step {step}"
            assert torch.equal(resid, ref_resid), f"tbq residual step {step}"
            subprocess.run([use_oracle, "tern_c", scratch.path("g.bin"), str(n), "2", "1", "1",
                            scratch.path("o.bin")], check=True)
            assert torch.equal(q, scratch.get("o.bin", np.uint8, 10 + n // 4)), f"terngrad step {step}"
            scratch.put("d.bin", torch.zeros(n))
            subprocess.run([use_oracle, "tern_d", scratch.path("o.bin"), str(10 + n // 4),
                            scratch.path("d.bin"), str(n), "0"], check=True)
            assert torch.equal(e, scratch.get("d.bin", np.float32, n)), f"terngrad decode step {step}"
    return {"tbq_payload": h_tbq.hexdigest(), "tbq_decoded": h_tbq_dec.hexdigest(),
            "terngrad_payload": h_tern.hexdigest(), "terngrad_decoded": h_tern_dec.hexdigest(),
            "torch": torch.__version__.split("+")[0]}


def test_roundtrip_config_against_reference(oracle, scratch):
    digests = _roundtrip_config_digests(oracle, scratch)
    if os.environ.get("HIPRESS_WRITE_GOLDEN"):
        os.makedirs(os.path.dirname(GOLDEN), exist_ok=True)
        with open(GOLDEN, "w") as f:
            json.dump(digests, f, indent=1)


def test_roundtrip_config_golden_digests():
    if not os.path.exists(GOLDEN):
        pytest.skip("golden digests not generated")
    golden = json.load(open(GOLDEN))
    if golden.get("torch") != torch.__version__.split("+")[0]:
        pytest.skip("golden digests were made with another torch RNG")
    digests = _roundtrip_config_digests()
    assert digests == golden
