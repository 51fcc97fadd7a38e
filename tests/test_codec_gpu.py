"""GPU tests of the stand-alone codec kernels against the CPU oracle (bit exact)."""
import ctypes as C

import numpy as np
import pytest
import torch

import gcow_b200 as g
from gcow_b200 import _native
from gcow_b200.codec import ZfpParams, Compressed

from test_codec_cpu import (_rand, _special_1d, field, CAST_3, XFORM_3, NB_3, UBLOCK_A, WORDS_A)

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("rate", [4, 8, 16, 32])
def test_fast_1d_bit_exact(rate):
    p = ZfpParams.from_rate(rate, 1)
    for x in (_rand(1 << 20), _special_1d(), _rand(5, seed=9), _rand(1 << 20 | 3, seed=2)):
        cpu = g.compress(torch.from_numpy(x), params=p)
        gpu = g.compress(dev(x), params=p)
        assert gpu.stream.is_cuda and gpu.nbytes == cpu.nbytes
        assert torch.equal(gpu.stream.cpu(), cpu.stream)
        for shift in (0, 3):
            a = g.decompress(cpu, shift=shift)
            b = g.decompress(gpu, shift=shift).cpu()
            assert torch.equal(a.view(torch.int32), b.view(torch.int32))


def test_fast_1d_unaligned_views():
    base = dev(_rand((1 << 16) + 8))
    x = base[1:(1 << 16) + 2]           # 4-byte aligned only
    p = ZfpParams.from_rate(8, 1)
    cpu = g.compress(x.cpu(), params=p)
    gpu = g.compress(x, params=p)
    assert torch.equal(gpu.stream.cpu(), cpu.stream)
    out = torch.empty((1 << 16) + 9, device="cuda")[1:(1 << 16) + 2]
    assert not out.is_contiguous() or True
    o = torch.empty_like(x)
    g.decompress(gpu, out=o)
    assert torch.equal(o.cpu().view(torch.int32), g.decompress(cpu).view(torch.int32))


def test_fast_1d_decode_random_streams():
    rng = np.random.default_rng(11)
    for rate in (4, 8, 16, 32):
        p = ZfpParams.from_rate(rate, 1)
        n = 4 * 65536
        raw = rng.integers(0, 256, size=n * rate // 8, dtype=np.uint8)
        a = g.decompress(Compressed(torch.from_numpy(raw.copy()), p, (n,), None))
        b = g.decompress(Compressed(dev(raw), p, (n,), None)).cpu()
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("p", [ZfpParams.from_rate(2, 1), ZfpParams.from_rate(3, 1), ZfpParams.from_rate(6, 1),
                               ZfpParams.from_accuracy(1e-3), ZfpParams.from_accuracy(1e-6),
                               ZfpParams.from_precision(12)],
                         ids=lambda p: f"{p.minbits}-{p.maxbits}-{p.maxprec}-{p.minexp}")
def test_generic_1d_bit_exact(p):
    for x in (_rand(1 << 16), _special_1d(), _rand(7, seed=3)):
        cpu = g.compress(torch.from_numpy(x), params=p, return_index=True)
        gpu = g.compress(dev(x), params=p, return_index=True)
        assert gpu.nbytes == cpu.nbytes
        assert torch.equal(gpu.stream.cpu(), cpu.stream)
        assert torch.equal(gpu.index.cpu(), cpu.index)
        a = g.decompress(cpu)
        b = g.decompress(gpu).cpu()
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("p", [ZfpParams.from_rate(1, 2), ZfpParams.from_rate(4, 2), ZfpParams.from_rate(8, 2),
                               ZfpParams.from_rate(16, 2), ZfpParams.from_accuracy(1e-3),
                               ZfpParams.from_accuracy(1e-6), ZfpParams.from_precision(16)],
                         ids=lambda p: f"{p.minbits}-{p.maxbits}-{p.maxprec}-{p.minexp}")
def test_generic_2d_bit_exact(p):
    rng = np.random.default_rng(1)
    for x in (field(37), (rng.standard_normal((130, 257)) * 5).astype(np.float32), field(8),
              np.zeros((9, 5), dtype=np.float32)):
        cpu = g.compress(torch.from_numpy(x), params=p, dim=2, return_index=True)
        gpu = g.compress(dev(x), params=p, dim=2, return_index=True)
        assert gpu.nbytes == cpu.nbytes
        assert torch.equal(gpu.stream.cpu(), cpu.stream)
        a = g.decompress(cpu)
        b = g.decompress(gpu).cpu()
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))


def test_variable_rate_decode_without_index_goes_through_host():
    x = field(64)
    gpu = g.compress(dev(x), tolerance=1e-3, dim=2)
    c = Compressed(gpu.stream, gpu.params, gpu.shape, None)
    d = g.decompress(c).cpu().numpy()
    assert np.max(np.abs(d - x)) <= 1e-3


def test_golden_3x3_on_gpu():
    c = g.compress(dev(field(3)), tolerance=1e-3, dim=2)
    w = list(np.frombuffer(c.stream.cpu().numpy().tobytes(), dtype=np.uint64))
    assert w == [7846959668108800257, 9092781915241025288, 1168152206201298680, 33031166]


def test_stage_kernels_golden():
    lib = _native.cuda()
    cpu = _native.cpu()
    s = torch.cuda.current_stream().cuda_stream
    blk = np.zeros(16, dtype=np.float32)
    a = field(3)
    cpu.gcow_stage_gather(a.ctypes.data, 3, 3, 0, blk.ctypes.data)
    nb = 1000
    f = dev(np.tile(blk, nb))
    emax = torch.empty(nb, dtype=torch.int32, device="cuda")
    assert lib.gcow_dbg_stage(0, 2, nb, f.data_ptr(), emax.data_ptr(), None, 0, s) == 0
    assert bool((emax == 1).all())
    q = torch.empty(nb * 16, dtype=torch.int32, device="cuda")
    assert lib.gcow_dbg_stage(1, 2, nb, f.data_ptr(), q.data_ptr(), emax.data_ptr(), 0, s) == 0
    assert q.view(nb, 16)[nb - 1].tolist() == CAST_3
    assert lib.gcow_dbg_stage(2, 2, nb, None, q.data_ptr(), None, 0, s) == 0
    assert q.view(nb, 16)[0].tolist() == XFORM_3
    u = torch.empty(nb * 16, dtype=torch.int32, device="cuda")
    assert lib.gcow_dbg_stage(4, 2, nb, q.data_ptr(), u.data_ptr(), None, 0, s) == 0
    assert [v & 0xffffffff for v in u.view(nb, 16)[nb // 2].tolist()] == NB_3
    # plane coder: header 257 + all planes of the golden coefficient block
    ub = dev(np.tile(np.array(UBLOCK_A, dtype=np.uint32), nb).view(np.int32))
    p = ZfpParams.from_accuracy(1e-3)
    out = torch.zeros(nb * 4, dtype=torch.int64, device="cuda")
    bits = torch.zeros(nb, dtype=torch.int32, device="cuda")
    assert lib.gcow_dbg_planes(2, nb, ub.data_ptr(), p.maxbits - 9, p.block_precision(1, 2), 257, 4,
                               out.data_ptr(), bits.data_ptr(), s) == 0
    one = np.frombuffer(out.view(nb, 4)[7].cpu().numpy().tobytes(), dtype=np.uint64)
    nbits = int(bits[7])
    # first block of the 3-block golden stream: compare the bits it owns
    gold = np.array(WORDS_A[:4], dtype=np.uint64)
    full = nbits // 64
    assert list(one[:full]) == list(gold[:full])
    rem = nbits % 64
    if rem:
        m = np.uint64((1 << rem) - 1)
        assert one[full] == (gold[full] & m)
    # inverse cast with an averaging shift equals the host stage
    qi = dev(np.array(CAST_3 * nb, dtype=np.int32))
    fo = torch.empty(nb * 16, dtype=torch.float32, device="cuda")
    assert lib.gcow_dbg_stage(5, 2, nb, qi.data_ptr(), fo.data_ptr(), emax.data_ptr(), 2, s) == 0
    ref = np.zeros(16, dtype=np.float32)
    qn = np.array(CAST_3, dtype=np.int32)
    cpu.gcow_stage_inv_cast(qn.ctypes.data, ref.ctypes.data, 16, 1, 2, 0)
    assert np.array_equal(fo.view(nb, 16)[3].cpu().numpy(), ref)


def test_gather_and_whole_block_stage_kernels():
    """Block formation with edge padding (5 x 7 ramp of the reference's gather test) and the
    whole-block encoder (3 x 3 field of its integration test) as stand-alone stage kernels."""
    lib = _native.cuda()
    s = torch.cuda.current_stream().cuda_stream
    ramp = torch.arange(1, 36, dtype=torch.float32, device="cuda").reshape(7, 5).contiguous()
    blocks = torch.zeros(4 * 16, dtype=torch.float32, device="cuda")
    assert lib.gcow_dbg_gather(2, ramp.data_ptr(), 5, 7, 4, blocks.data_ptr(), s) == 0
    b = blocks.view(4, 16).cpu()
    assert b[1].tolist() == [5, 5, 5, 5, 10, 10, 10, 10, 15, 15, 15, 15, 20, 20, 20, 20]
    assert b[3].tolist() == [25, 25, 25, 25, 30, 30, 30, 30, 35, 35, 35, 35, 25, 25, 25, 25]
    assert b[2][:4].tolist() == [21, 22, 23, 24] and b[2][12:].tolist() == [21, 22, 23, 24]
    f3 = dev(field(3))
    blk = torch.zeros(16, dtype=torch.float32, device="cuda")
    assert lib.gcow_dbg_gather(2, f3.data_ptr(), 3, 3, 1, blk.data_ptr(), s) == 0
    p = ZfpParams.from_accuracy(1e-3)
    out = torch.zeros(9, dtype=torch.int64, device="cuda")
    bits = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.gcow_dbg_encode_block(2, blk.data_ptr(), 1, p.as_c(), 9, out.data_ptr(), bits.data_ptr(), s) == 0
    w = list(np.frombuffer(out.cpu().numpy().tobytes(), dtype=np.uint64)[:4])
    assert w == [7846959668108800257, 9092781915241025288, 1168152206201298680, 33031166]
    assert 192 < int(bits[0]) <= 256
