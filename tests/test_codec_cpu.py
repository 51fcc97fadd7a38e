"""CPU tests of the codec: golden vectors taken from the reference's own tests,
oracle vs the header's fast formulation vs the reference build, round trips."""
import ctypes as C
import math
import os

import numpy as np
import pytest
import torch

import gcow_b200 as g
from gcow_b200 import _native
from gcow_b200.codec import ZfpParams

import refcodec

lib = _native.cpu()


def field(n):
    """exp(-(x^2+y^2)) on [0,2)^2, the reference's test input (sw/tests/test_zfp.cpp:13-25)."""
    a = np.zeros((n, n), dtype=np.float32)
    for j in range(n):
        for i in range(n):
            x = 2.0 * i / n
            y = 2.0 * j / n
            a[j, i] = np.float32(math.exp(-(x * x + y * y)))
    return a


def words(b):
    return list(np.frombuffer(b, dtype=np.uint64))


# ---------------------------------------------------------------- parameters
def test_params_modes():
    p = ZfpParams.from_accuracy(1e-3)
    assert (p.minbits, p.maxbits, p.maxprec, p.minexp) == (1, 16658, 64, -10)
    assert ZfpParams.from_rate(8, 1).maxbits == 32
    assert ZfpParams.from_rate(16, 1).maxbits == 64
    assert ZfpParams.from_rate(4, 1).maxbits == 16
    assert ZfpParams.from_rate(2, 1).maxbits == 9      # header floor
    assert ZfpParams.from_rate(8, 2).maxbits == 128
    assert ZfpParams.from_precision(12).maxprec == 12
    assert p.block_precision(1, 2) == 17 and p.block_precision(9, 2) == 25


def test_max_output_bytes_formula():
    p = ZfpParams.from_accuracy(1e-3)
    # 9 + 15 + 16*32 = 536 bits per 4x4 block, 148-bit header allowance
    assert g.max_compressed_nbytes((8, 8), p) == ((148 + 4 * 536 + 63) // 64) * 8


# -------------------------------------------------------------- stage goldens
CAST_3 = [536870912, 344231104, 90738336, 536870912, 344231104, 220714224, 58179640, 344231104,
          90738336, 58179640, 15335986, 90738336, 536870912, 344231104, 90738336, 536870912]
XFORM_3 = [264985681, 11130684, -112192135, 66784103, 11130684, 467543, -4712614, 2805257,
           -112192135, -4712614, 47500961, -28275684, 66784104, 2805256, -28275684, 16831537]
NB_3 = [282897489, 33434444, 33434444, 1796011, 156265097, 156265097, 13133998, 13133998,
        68099259, 68099256, 131453921, 8376857, 8376856, 38902892, 38902892, 16897137]


@pytest.mark.parametrize("which", [0, 1])
def test_stage_vectors_3x3(which):
    a = field(3)
    blk = np.zeros(16, dtype=np.float32)
    lib.gcow_stage_gather(a.ctypes.data, 3, 3, 0, blk.ctypes.data)
    # padded 3x3 block repeats row/col 0 in position 3
    assert blk[3] == blk[0] and blk[12] == blk[0] and blk[7] == blk[4]
    emax = lib.gcow_stage_emax(blk.ctypes.data, 16, which)
    assert emax == 1
    q = np.zeros(16, dtype=np.int32)
    lib.gcow_stage_cast(blk.ctypes.data, q.ctypes.data, 16, emax, which)
    assert list(q) == CAST_3
    lib.gcow_stage_xform(q.ctypes.data, 2, 0, which)
    assert list(q) == XFORM_3
    u = np.zeros(16, dtype=np.uint32)
    lib.gcow_stage_reorder(q.ctypes.data, u.ctypes.data, 2, which)
    assert list(u) == NB_3
    # inverses
    q2 = np.zeros(16, dtype=np.int32)
    lib.gcow_stage_inv_reorder(u.ctypes.data, q2.ctypes.data, 2, which)
    assert list(q2) == XFORM_3
    lib.gcow_stage_xform(q2.ctypes.data, 2, 1, which)
    assert np.max(np.abs(q2.astype(np.int64) - np.array(CAST_3))) <= 8  # lift is not exactly invertible


def test_gather_5x7_padding():
    # 5 wide, 7 tall ramp 1..35 -> 4 padded blocks (sw/tests/test_stages.cpp:147-167)
    a = np.arange(1, 36, dtype=np.float32).reshape(7, 5)
    blk = np.zeros(16, dtype=np.float32)
    lib.gcow_stage_gather(a.ctypes.data, 5, 7, 1, blk.ctypes.data)   # right edge: one column
    assert list(blk[:4]) == [5, 5, 5, 5] and list(blk[4:8]) == [10, 10, 10, 10]
    lib.gcow_stage_gather(a.ctypes.data, 5, 7, 2, blk.ctypes.data)   # bottom edge: 3 rows
    assert list(blk[:4]) == [21, 22, 23, 24] and list(blk[12:16]) == [21, 22, 23, 24]
    lib.gcow_stage_gather(a.ctypes.data, 5, 7, 3, blk.ctypes.data)
    assert list(blk) == [25, 25, 25, 25, 30, 30, 30, 30, 35, 35, 35, 35, 25, 25, 25, 25]


@pytest.mark.parametrize("which", [0, 1])
def test_stream_raw_writes(which):
    vals = (C.c_uint64 * 2)(7455816852505100291, 432)
    nb = (C.c_uint32 * 2)(64, 9)
    out = (C.c_uint64 * 4)()
    n = lib.gcow_stage_stream_write(vals, nb, 2, out, which)
    assert n == 2 and list(out[:2]) == [7455816852505100291, 432]


UBLOCK_A = [509992724, 444605396, 444605397, 118447768, 7401092, 7401093, 7263113, 7263112,
            29821528, 29821528, 73901, 29292361, 29292361, 300834, 300845, 1304446]
WORDS_A = [12711260835255415041, 5058120776611336133, 9096252834960252658, 7789501227241241664,
           10487902231007609841, 2274063208740063164, 6559061325237698320, 2621975557751902460,
           280285426033304047]


@pytest.mark.parametrize("which", [0, 1])
def test_encode_all_bitplanes_golden(which):
    # emax 1, tolerance 1e-3 -> maxprec 17; header 2*(1+127)+1 = 257; three copies
    u = np.array(UBLOCK_A, dtype=np.uint32)
    p = ZfpParams.from_accuracy(1e-3)
    prec = p.block_precision(1, 2)
    out = np.zeros(16, dtype=np.uint64)
    bits = lib.gcow_stage_encode_planes(u.ctypes.data, 16, p.maxbits - 9, prec, 257, 3,
                                        out.ctypes.data, which)
    assert list(out[:9]) == WORDS_A
    assert (bits + 63) // 64 == 9
    # decode the first copy back
    back = np.zeros(16, dtype=np.uint32)
    lib.gcow_stage_decode_planes(out.ctypes.data, 9, back.ctypes.data, 16, p.maxbits - 9, prec, which)
    mask = np.uint32((0xffffffff << (32 - prec)) & 0xffffffff)
    assert list(back) == list(u & mask)


IBLOCK = [6588397, 8685549, 10782701, 12879853, 216303600, 218400752, 220497904, 222595056,
          426018784, 428115936, 430213088, 432310240, 635734016, 637831168, 639928320, 642025472]


@pytest.mark.parametrize("which", [0, 1])
def test_encode_iblock_golden(which):
    # integer block, header value 2*9+1, tolerance 1e-3: precision 25, 95 payload bits, two words
    # (sw/tests/test_stages.cpp:742-789, hw/tests/test_encblock.cpp:166-183)
    p = ZfpParams.from_accuracy(1e-3)
    prec = p.block_precision(9, 2)
    assert prec == 25
    q = np.array(IBLOCK, dtype=np.int32)
    lib.gcow_stage_xform(q.ctypes.data, 2, 0, which)
    u = np.zeros(16, dtype=np.uint32)
    lib.gcow_stage_reorder(q.ctypes.data, u.ctypes.data, 2, which)
    out = np.zeros(4, dtype=np.uint64)
    bits = lib.gcow_stage_encode_planes(u.ctypes.data, 16, p.maxbits - 9, prec, 19, 1, out.ctypes.data, which)
    assert bits == 9 + 95
    assert list(out[:2]) == [72375632423897107, 1114129]


def test_whole_3x3_golden_words():
    # hw/tests/test_integration.cpp:166-174 == sw/tests/data/compressed_2d_3.zfp
    a = torch.from_numpy(field(3))
    c = g.compress(a, tolerance=1e-3, dim=2)
    assert words(c.stream.numpy().tobytes()) == [7846959668108800257, 9092781915241025288,
                                                 1168152206201298680, 33031166]


# ----------------------------------------------- oracle vs header vs reference
def _rand(n, scale=1e-3, seed=0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(n) * scale).astype(np.float32)


def _header_compress(x, p):
    nx, ny = (x.shape[1], x.shape[0]) if x.ndim == 2 else (x.size, 0)
    cap = g.max_compressed_nbytes(tuple(x.shape), p) + 16
    out = np.zeros(cap, dtype=np.uint8)
    n = lib.gcow_header_compress(x.ctypes.data, nx, ny, p.as_c(), out.ctypes.data)
    return out[:n].tobytes()


def _header_decompress(stream, shape, p, shift=0):
    nx, ny = (shape[1], shape[0]) if len(shape) == 2 else (shape[0], 0)
    buf = np.zeros(len(stream) + 16, dtype=np.uint8)
    buf[:len(stream)] = np.frombuffer(stream, dtype=np.uint8)
    out = np.zeros(shape, dtype=np.float32)
    lib.gcow_header_decompress(buf.ctypes.data, out.ctypes.data, nx, ny, p.as_c(), shift)
    return out


PARAM_SETS_1D = [ZfpParams.from_rate(r, 1) for r in (2, 3, 4, 8, 16, 32)] + \
    [ZfpParams.from_accuracy(t) for t in (1e-1, 1e-3, 1e-6, 1e-9)] + \
    [ZfpParams.from_precision(pr) for pr in (4, 12, 24, 32)]
PARAM_SETS_2D = [ZfpParams.from_rate(r, 2) for r in (1, 2, 4, 8, 16)] + \
    [ZfpParams.from_accuracy(t) for t in (1e-1, 1e-3, 1e-6)] + \
    [ZfpParams.from_precision(pr) for pr in (6, 16, 32)]


def _special_1d():
    x = _rand(4099)
    x[100:140] = 0.0                       # zero blocks
    x[200:204] = [1e-40, -3e-41, 0, 2e-45]  # subnormals
    x[300:304] = [1e-30, -1e-31, 1e-32, 0]  # below the cast's scale range
    x[400:404] = [3e38, -3e38, 1.0, 0.5]    # near float max
    x[500] = 123.456
    x[601:604] = [-1.0, 1.0, -1.0]
    return x


@pytest.mark.parametrize("p", PARAM_SETS_1D, ids=lambda p: f"{p.minbits}-{p.maxbits}-{p.maxprec}-{p.minexp}")
def test_1d_oracle_header_reference_agree(p):
    for x in (_rand(1 << 12), _special_1d(), _rand(7, seed=3), _rand(1, seed=4)):
        c = g.compress(torch.from_numpy(x), params=p, dim=1)
        s_or = c.stream.numpy().tobytes()
        s_hd = _header_compress(x, p)
        assert s_or == s_hd
        if refcodec.load() is not None:
            assert refcodec.compress(x, (p.minbits, p.maxbits, p.maxprec, p.minexp), 1) == s_or
        d_or = g.decompress(c).numpy()
        d_hd = _header_decompress(s_or, x.shape, p)
        assert np.array_equal(d_or.view(np.uint32), d_hd.view(np.uint32))
        if refcodec.load() is not None:
            d_rf = refcodec.decompress(s_or, x.shape, (p.minbits, p.maxbits, p.maxprec, p.minexp))
            assert np.array_equal(d_or.view(np.uint32), d_rf.view(np.uint32))


@pytest.mark.parametrize("p", PARAM_SETS_2D, ids=lambda p: f"{p.minbits}-{p.maxbits}-{p.maxprec}-{p.minexp}")
def test_2d_oracle_header_reference_agree(p):
    rng = np.random.default_rng(1)
    arrays = [field(37), (rng.standard_normal((13, 22)) * 5).astype(np.float32), field(8),
              np.zeros((9, 5), dtype=np.float32)]
    for x in arrays:
        c = g.compress(torch.from_numpy(x), params=p, dim=2)
        s_or = c.stream.numpy().tobytes()
        assert s_or == _header_compress(x, p)
        if refcodec.load() is not None:
            assert refcodec.compress(x, (p.minbits, p.maxbits, p.maxprec, p.minexp), 2) == s_or
        d_or = g.decompress(c).numpy()
        d_hd = _header_decompress(s_or, x.shape, p)
        assert np.array_equal(d_or.view(np.uint32), d_hd.view(np.uint32))
        if refcodec.load() is not None:
            d_rf = refcodec.decompress(s_or, x.shape, (p.minbits, p.maxbits, p.maxprec, p.minexp))
            assert np.array_equal(d_or.view(np.uint32), d_rf.view(np.uint32))


@pytest.mark.parametrize("rate", [4, 8, 16, 32])
def test_fast1d_matches_oracle(rate):
    p = ZfpParams.from_rate(rate, 1)
    for x in (_rand(1 << 14), _special_1d(), _rand(5, seed=9)):
        c = g.compress(torch.from_numpy(x), params=p, dim=1)
        blocks = (x.size + 3) // 4
        out = np.zeros(c.nbytes + 16, dtype=np.uint8)
        assert lib.gcow_fast1d_compress(x.ctypes.data, x.size, p.as_c(), out.ctypes.data) == 0
        nb = blocks * p.maxbits // 8
        assert out[:nb].tobytes() == c.stream.numpy().tobytes()[:nb]
        for shift in (0, 3):
            ref = g.decompress(c, shift=shift).numpy()
            got = np.zeros(x.size, dtype=np.float32)
            assert lib.gcow_fast1d_decompress(out.ctypes.data, got.ctypes.data, x.size, p.as_c(), shift) == 0
            assert np.array_equal(ref.view(np.uint32), got.view(np.uint32))


def _smooth_and_odd_1d():
    """Inputs that leave the warp-uniform fast path: smooth ramps and constants (the significance count stays
    below 3 for many planes), blocks whose members differ by many orders of magnitude, non-finite members, values
    below the cast's scale range and an all-tiny block whose coefficients have more than 24 leading zero planes."""
    rng = np.random.default_rng(11)
    parts = [np.linspace(-1.0, 1.0, 4096, dtype=np.float32),                        # ramp
             np.full(256, 0.3337, dtype=np.float32),                                # constant
             np.sin(np.arange(4096, dtype=np.float32) * 1e-3),                      # very smooth
             (rng.standard_normal(4096) * np.repeat(10.0 ** rng.integers(-12, 3, 1024), 4)).astype(np.float32),
             (rng.standard_normal(4096) * 10.0 ** rng.integers(-9, 1, 4096)).astype(np.float32),   # mixed within blocks
             np.array([1.0, 0, 0, 0, 0, 1.0, 0, 0, 0, 0, 1.0, 0, 0, 0, 0, 1.0], dtype=np.float32),
             np.array([1.0, 1.0, 1e-7, -1e-7, 1.0, -1.0, 3e-8, 0.0, 5.0, 5.0, 5.0, 5.0000005], dtype=np.float32),
             np.array([np.nan, 1.0, 2.0, 3.0, np.inf, 1.0, -1.0, 0.5, -np.inf, np.nan, 0.0, 1e-3,
                       1e-30, 2e-31, -3e-32, 1e-33, 1e-38, 1e-39, 0.0, -1e-40, -0.0, 0.0, -0.0, 0.0], dtype=np.float32)]
    return np.concatenate(parts)


@pytest.mark.parametrize("rate", [4, 8, 16, 32])
def test_lean_formulation_on_smooth_and_odd_data(rate):
    """gcow_fast1d_compress / _decompress run the three table-driven formulations on every block and fail (-2) if
    any two disagree; their common result must equal the serial oracle's."""
    p = ZfpParams.from_rate(rate, 1)
    with np.errstate(all="ignore"):
        xs = (_smooth_and_odd_1d(), _rand(1 << 18, seed=21), (_rand(1 << 16, seed=22) * 1e3).astype(np.float32))
    for x in xs:
        c = g.compress(torch.from_numpy(x), params=p, dim=1)
        blocks = (x.size + 3) // 4
        out = np.zeros(c.nbytes + 16, dtype=np.uint8)
        assert lib.gcow_fast1d_compress(x.ctypes.data, x.size, p.as_c(), out.ctypes.data) == 0
        nb = blocks * p.maxbits // 8
        assert out[:nb].tobytes() == c.stream.numpy().tobytes()[:nb]
        ref = g.decompress(c).numpy()
        got = np.zeros(x.size, dtype=np.float32)
        assert lib.gcow_fast1d_decompress(out.ctypes.data, got.ctypes.data, x.size, p.as_c(), 1) == 0
        assert np.array_equal(g.decompress(c, shift=1).numpy().view(np.uint32), got.view(np.uint32))
        assert ref.shape == x.shape


def test_fast1d_decoder_on_random_streams():
    # arbitrary bit patterns exercise budget exhaustion inside unary runs
    rng = np.random.default_rng(7)
    for rate in (4, 8, 16, 32):
        p = ZfpParams.from_rate(rate, 1)
        n = 4 * 4096
        raw = rng.integers(0, 256, size=n * rate // 8, dtype=np.uint8)
        # valid exponents only: keep the flag set and the biased exponent in a sane range
        c = g.codec.Compressed(torch.from_numpy(raw.copy()), p, (n,), None)
        ref = g.decompress(c).numpy()
        got = np.zeros(n, dtype=np.float32)
        assert lib.gcow_fast1d_decompress(raw.ctypes.data, got.ctypes.data, n, p.as_c(), 0) == 0
        assert np.array_equal(ref.view(np.uint32), got.view(np.uint32))
        hd = _header_decompress(raw.tobytes(), (n,), p)
        assert np.array_equal(ref.view(np.uint32), hd.view(np.uint32))


# ------------------------------------------------------------------ accuracy
def test_accuracy_mode_error_bound():
    x = field(64)
    for tol in (1e-1, 1e-3, 1e-6):
        c = g.compress(torch.from_numpy(x), tolerance=tol, dim=2)
        d = g.decompress(c).numpy()
        assert np.max(np.abs(d - x)) <= tol


def test_rate_mode_sizes_and_errors():
    x = _rand(1 << 20)
    xt = torch.from_numpy(x)
    expect_rmse = {4: 1.2e-3, 8: 8e-5, 16: 4e-7}
    for rate, lim in expect_rmse.items():
        c = g.compress(xt, rate=rate)
        assert c.nbytes == x.size * rate // 8
        d = g.decompress(c).numpy()
        rmse = float(np.sqrt(np.mean((d - x) ** 2)))
        assert rmse < lim
    c = g.compress(xt, rate=2)
    assert c.nbytes == ((x.size // 4 * 9 + 63) // 64) * 8


def test_shift_divides_exactly():
    x = _rand(1 << 10, scale=1.0)
    c = g.compress(torch.from_numpy(x), rate=16)
    a = g.decompress(c).numpy()
    b = g.decompress(c, shift=3).numpy()
    assert np.array_equal(a / 8, b)


# -------------------------------------------------------------- golden files
GOLDEN_SIZES = [3, 8, 100, 123, 210, 345, 354, 500, 505, 510]


@pytest.mark.parametrize("n", GOLDEN_SIZES)
def test_reference_golden_files(n):
    path = refcodec.REF / "sw" / "tests" / "data" / f"compressed_2d_{n}.zfp"
    if not path.exists():
        pytest.skip("reference checkout not present")
    c = g.compress(torch.from_numpy(field(n)), tolerance=1e-3, dim=2)
    assert c.stream.numpy().tobytes() == path.read_bytes()


def test_cli_matches_golden_and_prints(tmp_path, capsys):
    """The command-line counterpart of the reference host program: generate the field, compress at tolerance 1e-3,
    write the stream, compare with the golden file, print a corner of the field and the first stream words."""
    from gcow_b200 import cli
    path = refcodec.REF / "sw" / "tests" / "data" / "compressed_2d_100.zfp"
    if not path.exists():
        pytest.skip("reference checkout not present")
    out = tmp_path / "c.gcow"
    rc = cli.main(["100", "--device", "cpu", "--golden", str(path), "--out", str(out), "--print", "2", "--iters", "1",
                   "--roundtrip"])
    assert rc == 0 and out.read_bytes() == path.read_bytes()
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 4 and lines[0].split()[0].startswith("1.0")          # field(0, 0) = exp(0)
    assert len(lines[2].split()) == 2 and all(len(w) == 16 for w in lines[2].split())
    import json
    rep = json.loads(lines[3])
    assert rep["golden_match"] and rep["max_abs_error"] < 1e-3
    padded = tmp_path / "p.gcow"
    assert cli.main(["100", "--device", "cpu", "--out", str(padded), "--pad64", "--iters", "1"]) == 0
    assert len(padded.read_bytes()) % 64 == 0


def test_cli_reads_a_raw_float32_field(tmp_path, capsys):
    """A header-less float32 dump with --shape, as the reference's data probe reads its climate field
    (hw/tests/parse_dat.cpp:1-38): same stream as the same array given as .npy."""
    import json
    from gcow_b200 import cli
    a = field(36)[:20]                                   # 20 rows x 36 columns
    raw, npy = tmp_path / "f.dat", tmp_path / "f.npy"
    a.astype("<f4").tofile(raw)
    np.save(npy, a)
    o1, o2 = tmp_path / "a.gcow", tmp_path / "b.gcow"
    assert cli.main(["--input", str(raw), "--shape", "20", "36", "--device", "cpu", "--out", str(o1), "--iters", "1",
                     "--print", "3"]) == 0
    first = capsys.readouterr().out.strip().splitlines()
    assert first[0].split()[0].startswith("1.0") and json.loads(first[-1])["values"] == 720
    assert cli.main(["--input", str(npy), "--device", "cpu", "--out", str(o2), "--iters", "1"]) == 0
    assert o1.read_bytes() == o2.read_bytes()


@pytest.mark.parametrize("bits", [16, 32, 64, 128])
@pytest.mark.parametrize("tol", [1e-1, 1e-2, 1e-3, 1e-6, 1e-9])
def test_lean_coders_under_the_accuracy_rule(bits, tol):
    """Fixed accuracy with a bit cap on the lean (table-driven) coders, as the sparse all-reduce uses them, against
    the plane-by-plane definition: noise, quantised values (few planes set), smooth ramps, tiny and huge blocks."""
    import ctypes as C
    from gcow_b200 import _native
    rng = np.random.default_rng(bits)
    n = 40000
    minexp = ZfpParams.from_accuracy(tol).minexp
    cases = [
        rng.standard_normal(n) * 1e-3,
        np.round(rng.standard_normal(n) * 8) / 8 * 1e-3,             # few significant planes
        np.linspace(0, 1e-2, n),                                     # smooth
        rng.standard_normal(n) * 10.0 ** rng.integers(-12, 3, n),    # every magnitude
        np.where(rng.random(n) < 0.7, 0.0, rng.standard_normal(n)),  # mostly zeros
    ]
    for x in cases:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        bad = _native.cpu().gcow_lean_accuracy_check(x.ctypes.data, n, bits, minexp, out.ctypes.data)
        assert bad == 0
        kept = np.abs(out).reshape(-1, 4).max(axis=1) > 0
        if kept.any() and bits == 128 and tol >= 1e-3 and np.abs(x).max() < 1:   # where the cap never cuts, the bound holds
            assert np.abs(out - x).max() <= tol
