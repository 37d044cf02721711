"""Pins both CPU oracles (torch-op port and C restatement) to golden vectors
produced by the real reference modules (tests/golden/make_golden.py), and to
the known-answer vectors the reference's own tests hold.  CPU only."""

import numpy as np
import pytest
import torch

from oracle import cref, ref_port

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _bf16(u16):
    return torch.from_numpy(u16.view(np.int16).copy()).view(torch.bfloat16)


def test_tables_match_reference(golden):
    t = golden("tables")
    assert t["values"].tolist() == E2M1 + [-v for v in E2M1]
    assert t["e4m3"][:8].tolist() == list(ref_port.E2M1_E4M3)
    assert t["e4m3"][8:].tolist() == [b | 0x80 for b in ref_port.E2M1_E4M3]
    assert t["q"].tolist() == [int(2 * v) for v in t["values"]]
    # reference tests/test_fp4.py:48-51: midpoints keep the smaller magnitude
    assert t["mid_codes"].tolist() == [0, 1, 2, 3, 4, 5, 6]
    assert t["neg_mid_codes"].tolist() == [8, 9, 10, 11, 12, 13, 14]
    mids = torch.from_numpy(t["mids"])
    assert ref_port.round_e2m1(mids).tolist() == [0, 1, 2, 3, 4, 5, 6]
    assert ref_port.round_e2m1(mids, "rne").tolist() == [0, 2, 2, 4, 4, 6, 6]


def test_e4m3_known_answer_word():
    # reference cuda/test_unpack.c:26: nibbles of 0xFEDCBA98 expand to these bytes
    word = 0xFEDCBA98
    nib = [(word >> (4 * i)) & 0xF for i in range(8)]
    tbl = list(ref_port.E2M1_E4M3) + [b | 0x80 for b in ref_port.E2M1_E4M3]
    by = bytes(tbl[n] for n in nib)
    assert by[:4][::-1].hex() == "bcb8b080" and by[4:][::-1].hex() == "ccc8c4c0"


@pytest.mark.parametrize("name", ["quant_adversarial_f32"])
def test_quantize_adversarial(golden, name):
    gd = golden(name)
    x = gd["x"].view(np.float32)
    codes, scale = ref_port.quantize(torch.from_numpy(x.copy()))
    assert np.array_equal(codes.numpy(), gd["codes"])
    assert np.array_equal(scale.numpy().view(np.uint32), gd["scale"])
    assert np.array_equal(ref_port.pack(codes).numpy(), gd["packed"])
    c = cref.quantize(x)
    assert np.array_equal(c["codes"], gd["codes"])
    assert np.array_equal(c["scale"].view(np.uint32), gd["scale"])
    assert np.array_equal(c["packed"], gd["packed"])
    e = ((gd["scale"] >> 23) & 0xFF).astype(np.uint8)
    assert np.array_equal(c["e8m0"], e)


def test_quantize_nan_block(golden):
    gd = golden("quant_nan_f32")
    x = gd["x"].view(np.float32)
    codes, scale = ref_port.quantize(torch.from_numpy(x.copy()))
    assert np.array_equal(codes.numpy(), gd["codes"])
    gs = gd["scale"].view(np.float32)
    assert np.array_equal(np.isnan(scale.numpy()), np.isnan(gs))
    c = cref.quantize(x)
    assert np.array_equal(np.isnan(c["scale"]), np.isnan(gs))
    ok = ~np.isnan(gs)
    assert np.array_equal(c["scale"][ok], gs[ok])
    blk_ok = np.repeat(ok, 32, axis=-1)
    assert np.array_equal(c["codes"][blk_ok], gd["codes"][blk_ok])
    # in a NaN block the reference gives magnitude 7 everywhere
    assert ((gd["codes"][~blk_ok] & 7) == 7).all()
    assert ((c["codes"][~blk_ok] & 7) == 7).all()


def test_quantize_bf16_and_gemm(golden):
    gd = golden("quant_gemm_bf16")
    a, w = _bf16(gd["a"]), _bf16(gd["w"])
    ac, asc = ref_port.quantize(a)
    wc, wsc = ref_port.quantize(w)
    assert np.array_equal(ac.numpy(), gd["a_codes"]) and np.array_equal(asc.numpy(), gd["a_scale"])
    assert np.array_equal(wc.numpy(), gd["w_codes"]) and np.array_equal(wsc.numpy(), gd["w_scale"])
    assert np.array_equal(ref_port.pack(ac).numpy(), gd["a_packed"])
    assert np.array_equal(ref_port.unpack(ref_port.pack(ac)).numpy(), gd["a_codes"])
    assert np.array_equal(ref_port.dequantize(ac, asc).numpy(), gd["a_deq"])
    c16, s16 = ref_port.quantize(a, 16)
    assert np.array_equal(c16.numpy(), gd["a_codes16"]) and np.array_equal(s16.numpy(), gd["a_scale16"])
    # C restatement
    c = cref.quantize(a.float().numpy())
    assert np.array_equal(c["codes"], gd["a_codes"]) and np.array_equal(c["scale"], gd["a_scale"])
    assert np.array_equal(c["packed"], gd["a_packed"])
    assert np.array_equal(cref.unpack(gd["a_packed"]), gd["a_codes"])
    assert np.array_equal(cref.pack(gd["a_codes"]), gd["a_packed"])
    assert np.array_equal(cref.dequantize(gd["a_codes"], gd["a_scale"]), gd["a_deq"])
    c = cref.quantize(a.float().numpy(), block=16)
    assert np.array_equal(c["codes"], gd["a_codes16"]) and np.array_equal(c["scale"], gd["a_scale16"])
    # GEMM: same torch sgemm -> equal up to thread-count blocking; hold to 1 bf16 ulp
    out = ref_port.gemm_fake_quant(ac, asc, wc, wsc)
    want = _bf16(gd["out_bf16"])
    assert (out.float() - want.float()).abs().max() <= want.float().abs().max() * 2 ** -7
    ref64 = ref_port.gemm_fp64(ac, asc, wc, wsc)
    assert torch.allclose(ref64.float(), torch.from_numpy(gd["out_ref_f32"]), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("block", [16, 32])
def test_quantize_logspace(golden, block):
    gd = golden(f"quant_logspace_b{block}")
    codes, scale = ref_port.quantize(torch.from_numpy(gd["x"]), block)
    assert np.array_equal(codes.numpy(), gd["codes"]) and np.array_equal(scale.numpy(), gd["scale"])
    c = cref.quantize(gd["x"], block=block)
    assert np.array_equal(c["codes"], gd["codes"]) and np.array_equal(c["scale"], gd["scale"])
    # properties the reference's own test asserts (tests/test_fp4.py:54-68)
    s = torch.from_numpy(c["scale"])
    assert torch.equal(torch.exp2(torch.log2(s).round()), s)
    amax = np.abs(gd["x"]).reshape(64, -1, block).max(-1)
    assert ((amax / c["scale"] >= 4 * (1 - 1e-6)) & (amax / c["scale"] < 8)).all()


def test_block_exponent_rule_equals_torch_log2():
    """The integer rule of the C oracle (and of the CUDA kernels) against
    torch.floor(torch.log2(.)) in fp32 on every exponent x the 64 values
    below each power of two, plus random fp32 values."""
    vals = []
    for k in range(-100, 128):
        top = np.array([2.0 ** k], np.float32).view(np.uint32)[0]
        for n in range(0, 64):
            vals.append(top - n)
    rng = np.random.default_rng(0)
    rnd = rng.integers(0x0D000000, 0x7F7FFFFF, 200_000, dtype=np.uint32)
    u = np.concatenate([np.array(vals, np.uint32), rnd])
    a = u.view(np.float32)
    a = a[a >= 1e-30]
    want = (torch.floor(torch.log2(torch.from_numpy(a.copy()))) - 2).clamp(-127, 127).numpy()
    got = np.array([cref.block_exponent(v) for v in a[:20000]], np.float32)
    assert np.array_equal(got, want[:20000])
    # the rest through the vectorised path: one element per block decides E
    x = np.zeros((a.size, 32), np.float32)
    x[:, 0] = a
    c = cref.quantize(x, want=("e8m0",))
    assert np.array_equal(c["e8m0"][:, 0].astype(np.float32) - 127, want)


def test_linear_golden(golden):
    gd = golden("linear_ste")
    w = torch.from_numpy(gd["w"])
    x, gy = _bf16(gd["x"]), _bf16(gd["gy"])
    y = ref_port.linear_forward(x.reshape(-1, 256), w)
    want = _bf16(gd["y"]).reshape(-1, 160)
    assert (y.float() - want.float()).abs().max() <= want.float().abs().max() * 2 ** -7
    gx, gw = ref_port.linear_backward_ste(gy.reshape(-1, 160), x.reshape(-1, 256), w)
    assert torch.allclose(gx.float(), _bf16(gd["gx"]).reshape(-1, 256).float(), rtol=2e-2, atol=1e-2)
    assert torch.allclose(gw, torch.from_numpy(gd["gw"]), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("method,lim,ef", [("int16", 32767, False), ("int8", 127, False),
                                            ("int8ef", 127, True)])
def test_integer_wire_golden(golden, method, lim, ef):
    gd = golden(f"wire_{method}_w1")
    g = torch.from_numpy(gd["g"])
    padded = ref_port.padded_len(g.numel(), 1)
    res = [torch.zeros(padded)] if ef else None
    ores = [torch.zeros(padded // 64, 64)] if ef else None
    for s in range(3):
        out = ref_port.wire_int_step([g * (1 + 0.5 * s)], lim, res, ores)[0]
        assert np.array_equal(out.numpy(), gd["outs"][s]), (method, s)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("method,lim,ef", [("int16", 32767, False), ("int8", 127, False),
                                            ("int8ef", 127, True)])
def test_integer_wire_golden_several_ranks(golden, method, lim, ef, world):
    # outputs of the real reference Wire on 2 and 4 gloo ranks (make_golden_wire_ranks.py)
    gd = golden(f"wire_{method}_w{world}")
    grads = gd["grads"]                                      # [step, rank, n]
    n = grads.shape[-1]
    padded = ref_port.padded_len(n, world)
    res = [torch.zeros(padded) for _ in range(world)] if ef else None
    ores = [torch.zeros(padded // 64 // world, 64) for _ in range(world)] if ef else None
    for s in range(3):
        outs = ref_port.wire_int_step([torch.from_numpy(grads[s, r].copy()) for r in range(world)], lim, res, ores)
        for r in range(world):
            assert np.array_equal(outs[r].numpy(), gd["outs"][s]), (method, world, s, r)


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("ef", [False, True])
def test_mxfp4_wire_golden(golden, world, ef):
    gd = golden(f"wire_mxfp4{'ef' if ef else ''}_w{world}")
    grads = gd["grads"]                      # [step, rank, n]
    n = grads.shape[-1]
    padded = ref_port.padded_len(n, world)
    shard = padded // world
    res_t = [torch.zeros(padded) for _ in range(world)] if ef else None
    ores_t = [torch.zeros(shard) for _ in range(world)] if ef else None
    res_c = [np.zeros(padded, np.float32) for _ in range(world)] if ef else None
    ores_c = [np.zeros(shard, np.float32) for _ in range(world)] if ef else None
    for step in range(3):
        gs = [torch.from_numpy(grads[step, r]) for r in range(world)]
        outs, sent, owned = ref_port.wire_mxfp4_step(gs, res_t, ores_t, return_bytes=True)
        out_c, sent_c, owned_c = cref.wire_step([grads[step, r] for r in range(world)], res_c, ores_c)
        for r in range(world):
            assert np.array_equal(sent[r][0].numpy(), gd[f"sent_p{step}"][r])
            assert np.array_equal(sent[r][1].numpy(), gd[f"sent_e{step}"][r])
            assert np.array_equal(sent_c[r][0], gd[f"sent_p{step}"][r])
            assert np.array_equal(sent_c[r][1], gd[f"sent_e{step}"][r])
        assert np.array_equal(torch.cat([p for p, _ in owned]).numpy(), gd[f"own_p{step}"])
        assert np.array_equal(np.concatenate([p for p, _ in owned_c]), gd[f"own_p{step}"])
        assert np.array_equal(np.concatenate([e for _, e in owned_c]), gd[f"own_e{step}"])
        assert np.array_equal(outs[0].numpy(), gd[f"out{step}"])
        assert np.array_equal(out_c, gd[f"out{step}"])


def test_dual_slot_split():
    # reference tests/test_fp4.py:95-102
    for k in (8, 32, 128):
        s = ref_port.slot_offset(k)
        c1 = torch.tensor([144.0 * k, -144.0 * k, 3.0], dtype=torch.float64)
        c2 = torch.tensor([-144.0 * k, 144.0 * k, -7.0], dtype=torch.float64)
        g1, g2 = ref_port.unpack_dual(c1 + c2 * 2.0 ** s, s)
        assert torch.equal(g1, c1) and torch.equal(g2, c2)


@pytest.mark.parametrize("world", [3, 5, 6, 7])
def test_c_oracle_equals_torch_port_for_odd_worlds(world):
    """The final division by the world size: torch divides a tensor by a scalar as
    x * (1 / world) (wire.py:138 `.div_(world)`); not exact unless world is a power
    of two, so the C restatement must do the same."""
    rng = np.random.default_rng(world)
    gs = [(rng.standard_t(3, 3000) * 1e-3).astype(np.float32) for _ in range(world)]
    out_c, _, _ = cref.wire_step(gs)
    out_t = ref_port.wire_mxfp4_step([torch.from_numpy(g) for g in gs])[0].numpy()
    assert np.array_equal(out_c, out_t)
