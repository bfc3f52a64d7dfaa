"""Bit-exactness of code expansion and dequantisation on the GPU (through the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import qgemv_oracle as O
from ai_accel_studio_b200 import ops
from ai_accel_studio_b200.kernels.groupwise_int2 import GroupwiseInt2Weight, pack_groupwise_int2, unpack_groupwise_int2, unpack_codes_int2
from ai_accel_studio_b200.kernels.groupwise_int4 import GroupwiseInt4Weight, pack_groupwise_int4, unpack_groupwise_int4, unpack_codes_int4

pytestmark = pytest.mark.gpu


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def test_codes_and_dequant_match_fixtures(small_cases):
    z, meta = small_cases
    for c in meta["pack_cases"]:
        nm = c["name"]
        packed = torch.from_numpy(z[nm + ".packed"]).cuda()
        scales = torch.from_numpy(z[nm + ".scales"]).cuda()
        cls, unpack, codes_fn, ocodes = (GroupwiseInt2Weight, unpack_groupwise_int2, unpack_codes_int2, O.unpack_codes_int2) \
            if c["bits"] == 2 else (GroupwiseInt4Weight, unpack_groupwise_int4, unpack_codes_int4, O.unpack_codes_int4)
        pw = cls(packed, scales, c["original_k"], c["padded_k"], c["group"])
        assert np.array_equal(codes_fn(pw).cpu().numpy(), ocodes(z[nm + ".packed"])), nm
        d32 = unpack(pw, torch.float32).cpu().numpy()
        d16 = unpack(pw, torch.float16).cpu().numpy()
        assert d32.shape == (c["n"], c["k"])
        assert np.array_equal(_bits(d32), _bits(z[nm + ".deq32"])), nm   # what the reference's torch code produced
        assert np.array_equal(_bits(d16), _bits(z[nm + ".deq16"])), nm


@pytest.mark.parametrize("bits,n,k,group", [(2, 300, 1024, 64), (2, 257, 4096, 128), (4, 129, 2048, 128), (4, 64, 896, 128),
                                            (2, 3, 12, 4), (4, 5, 6, 2)])
def test_dequant_random_all_dtypes(bits, n, k, group):
    g = torch.Generator().manual_seed(bits * 1000 + n)
    w = torch.randn(n, k, generator=g) * 0.03
    pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(w, group)
    host = O.PackedWeight(bits, pw.packed.numpy(), pw.scales.numpy(), pw.original_k, pw.padded_k, group)
    dev = type(pw)(pw.packed.cuda(), pw.scales.cuda(), pw.original_k, pw.padded_k, group)
    unpack = unpack_groupwise_int2 if bits == 2 else unpack_groupwise_int4
    assert np.array_equal(_bits(unpack(dev, torch.float32).cpu().numpy()), _bits(O.dequant(host, np.float32)))
    assert np.array_equal(_bits(unpack(dev, torch.float16).cpu().numpy()), _bits(O.dequant(host, np.float16)))
    # bfloat16: compare with the torch expression of the reference evaluated on the host
    codes = torch.from_numpy(O.unpack_codes(host).astype(np.int64))
    if bits == 2:
        vals = torch.tensor(O.INT2_LEVELS_F32.tolist(), dtype=torch.float64).to(torch.bfloat16)
        vals = torch.tensor((-1.0, -1.0 / 3.0, 1.0 / 3.0, 1.0), dtype=torch.bfloat16)[codes]
    else:
        vals = (codes.to(torch.int16) - 8).to(torch.bfloat16)
    gids = torch.arange(pw.padded_k) // group
    want = (vals * pw.scales.to(torch.bfloat16)[:, gids])[:, :pw.original_k]
    got = unpack(dev, torch.bfloat16).cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_padded_tail_is_dropped_and_codes_keep_it():
    w = torch.randn(9, 130)
    pw = pack_groupwise_int2(w, 64)
    dev = GroupwiseInt2Weight(pw.packed.cuda(), pw.scales.cuda(), 130, 192, 64)
    assert tuple(unpack_groupwise_int2(dev).shape) == (9, 130)
    assert tuple(unpack_codes_int2(dev).shape) == (9, 192)


def test_dequant_rejects_cpu():
    pw = pack_groupwise_int4(torch.randn(4, 64), 32)
    with pytest.raises(RuntimeError, match="CUDA"):
        unpack_groupwise_int4(pw)
