"""The reference-signature entry points of dual_gemm (bf16 / fp8 operands on the
FP4 integer grid, fp32 out) on the GPU: dual_gemm.py:215-289, and the slot
split pinned by the reference's tests/test_fp4.py:95-102.  Operands hold
q = 2 * value, so every product and sum is an integer and the expected result
is exact: fp64 matmul of the same operands."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dg():
    from lockstep_b200 import dual_gemm
    return dual_gemm


def _q(shape, seed, dtype):
    from lockstep_b200 import fp4
    g = torch.Generator(device="cuda").manual_seed(seed)
    codes = torch.randint(0, 16, shape, dtype=torch.uint8, device="cuda", generator=g)
    return fp4.codes_to_q(codes).to(dtype)                 # integers in [-12, 12]


def test_dual_slot_split(dg):
    # the reference's own test, on the device
    for k in (8, 32, 128):
        s = dg.slot_offset(k)
        c1 = torch.tensor([144.0 * k, -144.0 * k, 3.0], dtype=torch.float64, device="cuda")
        c2 = torch.tensor([-144.0 * k, 144.0 * k, -7.0], dtype=torch.float64, device="cuda")
        g1, g2 = dg.unpack_dual(c1 + c2 * 2.0 ** s, s)
        assert torch.equal(g1, c1) and torch.equal(g2, c2)
    assert [dg.slot_offset(k) for k in (8, 14, 64, 4096)] == [12, 12, 15, 21]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 136, 512), (64, 64, 4096)])
def test_gemm_and_dual_separate_exact(dg, dtype, M, N, K):
    a1, a2 = _q((M, K), 1, dtype), _q((M, K), 2, dtype)
    b1, b2 = _q((K, N), 3, dtype), _q((K, N), 4, dtype)
    want1 = a1.double() @ b1.double()
    want2 = a2.double() @ b2.double()
    c = dg.gemm(a1, b1)
    assert c.dtype == torch.float32 and torch.equal(c.double(), want1)
    c1, c2 = dg.dual_separate(a1, a2, b1, b2)
    assert torch.equal(c1.double(), want1) and torch.equal(c2.double(), want2)
    s1, s2 = dg.splitk_separate(a1, a2, b1, b2, splits=K // 64 if K // 64 <= 8 else 8)
    assert torch.equal(s1.double(), want1) and torch.equal(s2.double(), want2)
    # shared weight, as train_step.py:52-53 calls it
    c1, c2 = dg.dual_separate(a1, a2, b1, b1)
    assert torch.equal(c1.double(), want1) and torch.equal(c2.double(), a2.double() @ b1.double())


def test_dual_packed_round_trip_small_k(dg):
    # The packed accumulator C1 + 2^s C2 is exact in fp32 only while
    # 2 * bits(144 K) + 1 <= 24 (dual_gemm.py:10-15): K <= 14, reached by zero padding to 64
    k_real, K, M, N = 8, 64, 128, 128
    s = dg.slot_offset(k_real)
    a1, a2 = _q((M, K), 5, torch.bfloat16), _q((M, K), 6, torch.bfloat16)
    b1, b2 = _q((K, N), 7, torch.bfloat16), _q((K, N), 8, torch.bfloat16)
    for t in (a1, a2):
        t[:, k_real:] = 0
    acc = dg.dual_packed(a1, (a2.float() * 2.0 ** s).to(torch.float32), b1, b2)
    g1, g2 = dg.unpack_dual(acc, s)
    assert torch.equal(g1.double(), a1.double() @ b1.double())
    assert torch.equal(g2.double(), a2.double() @ b2.double())
    sp = dg.splitk_packed(a1, (a2.float() * 2.0 ** s), b1, b2, splits=1)
    assert torch.equal(sp, acc)


def test_preconditions_are_assertions(dg):
    a, b = _q((128, 96), 1, torch.bfloat16), _q((96, 64), 2, torch.bfloat16)
    with pytest.raises(AssertionError):
        dg.gemm(a, b)                                       # K % 64
    with pytest.raises(AssertionError):
        dg.dual_separate(a, a, b, b)
    a, b = _q((128, 192), 1, torch.bfloat16), _q((192, 64), 2, torch.bfloat16)
    with pytest.raises(AssertionError):
        dg.splitk_separate(a, a, b, b, splits=2)            # K % (splits * 64)
    with pytest.raises(RuntimeError):
        dg.gemm(a.cpu(), b.cpu())                           # no CPU path
