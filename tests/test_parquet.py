"""The native Parquet decoder (reference: io/parquet/parquet_test.go).  Three sources of truth: the
reference's fixture files with the closed-form value of every row (parquet_test.go:38-75), files
written here by pyarrow with every encoding / codec / page version the decoder knows, and damaged
files that must be refused with an error, never a crash."""
import math
import os
import struct

import numpy as np
import pytest
import torch

from mimir_b200.io import parquet
from tests._refdir import reference_dir

pa = pytest.importorskip("pyarrow")
pq = pytest.importorskip("pyarrow.parquet")


# ------------------------------------------------------------------ reference fixtures
FIXTURES = {
    "plain_v1": (1000, [1000]), "dict_v1_snappy": (1000, [1000]), "dict_v2_gzip": (1000, [1000]),
    "dict_v2_zstd": (1000, [1000]), "delta_v2": (1000, [1000]), "delta_byte_array_v2": (1000, [1000]),
    "pages_v2_snappy": (10000, [4000, 4000, 2000]), "empty": (0, [0]),
}


def _fixture(name):
    root = reference_dir()
    path = os.path.join(root, "io", "parquet", "testdata", name + ".parquet") if root else None
    if not path or not os.path.exists(path):
        pytest.skip("reference fixtures not present")
    return path


@pytest.mark.parametrize("name", sorted(FIXTURES))
def test_reference_fixture_values_follow_their_formulas(name):
    rows, groups = FIXTURES[name]
    f = parquet.File(_fixture(name))
    assert f.rows == rows and f.row_groups == len(groups)
    assert f.columns == ["i32", "i64", "f32", "f64", "flag", "name", "opt"]
    info = {c.name: c for c in f.column_info()}
    assert [info[c].type for c in f.columns] == [parquet.INT32, parquet.INT64, parquet.FLOAT, parquet.DOUBLE, parquet.BOOLEAN,
                                                 parquet.BYTE_ARRAY, parquet.FLOAT]
    assert all(info[c].nullable and not info[c].nested for c in f.columns) and info["name"].logical == "STRING"
    assert f.created_by.startswith("parquet-cpp-arrow") and "ARROW:schema" in f.metadata()
    start = 0
    for g, n in enumerate(groups):
        assert f.row_group_rows(g) == n
        i = np.arange(start, start + n, dtype=np.int64)
        v, nulls = f.read_column(g, "i32")
        assert v.dtype == torch.int32 and not nulls.any() and np.array_equal(v.numpy(), (7 * i - 100).astype(np.int32))
        v, nulls = f.read_column(g, "i64")
        assert np.array_equal(v.numpy(), i * 10_000_000_000 - 5) and not nulls.any()
        v, _ = f.read_column(g, "f32")
        assert np.array_equal(v.numpy(), (i.astype(np.float64) / 3).astype(np.float32))
        v, _ = f.read_column(g, "f64")
        assert np.array_equal(v.numpy(), np.sqrt(i.astype(np.float64)))
        v, _ = f.read_column(g, "flag")
        assert v.dtype == torch.bool and np.array_equal(v.numpy(), i % 3 == 0)
        v, _ = f.read_column(g, "name")
        assert v == ["s%d" % (k % 17) for k in i]
        v, nulls = f.read_column(g, "opt")
        assert np.array_equal(nulls.numpy(), i % 5 == 0)
        want = np.where(i % 5 == 0, 0, (i.astype(np.float64) / 2)).astype(np.float32)
        assert np.array_equal(v.numpy(), want)
        start += n
    whole = f.read()
    if rows:
        assert whole["opt"].shape == (rows,) and bool(torch.isnan(whole["opt"][0])) and float(whole["opt"][1]) == 0.5
    with pytest.raises(KeyError):
        f.column("nope")
    with pytest.raises(IndexError):
        f.read_column(len(groups), "i32")


# ------------------------------------------------------------------ files written here
def _table(n, seed=0):
    rng = np.random.default_rng(seed)
    i = np.arange(n)
    opt = [None if k % 7 == 0 else float(k) / 4 for k in i]
    words = ["alpha", "beta", "", "gamma-" * 9, "δέλτα"]
    return {
        "i32": pa.array((rng.integers(-2**31, 2**31, n)).astype(np.int32)),
        "i64": pa.array(rng.integers(-2**62, 2**62, n).astype(np.int64)),
        "seq": pa.array((1000 + 3 * i).astype(np.int64)),
        "f32": pa.array(rng.standard_normal(n).astype(np.float32)),
        "f64": pa.array(rng.standard_normal(n)),
        "flag": pa.array(i % 3 == 0),
        "cat": pa.array([words[k % 5] for k in i]),
        "uniq": pa.array(["row-%06d" % k for k in i]),
        "blob": pa.array([bytes([k % 251]) * (k % 9) for k in i], pa.binary()),
        "fix": pa.array([struct.pack("<I", int(k)) for k in i], pa.binary(4)),
        "opt": pa.array(opt, pa.float64()),
        "opt_s": pa.array([None if k % 4 == 1 else "v%d" % (k % 11) for k in i]),
        "opt_i": pa.array([None if k % 6 == 2 else int(k) - 50 for k in i], pa.int32()),
        "all_null": pa.array([None] * n, pa.float32()),
    }


def _check_against_arrow(path, groups_expected=None):
    f = parquet.File(path)
    ref = pq.ParquetFile(path)
    assert f.rows == ref.metadata.num_rows and f.row_groups == ref.metadata.num_row_groups
    if groups_expected is not None:
        assert f.row_groups == groups_expected
    for g in range(f.row_groups):
        tbl = ref.read_row_group(g)
        for name in tbl.column_names:
            want = tbl.column(name).to_pylist()
            got, nulls = f.read_column(g, name)
            if torch.is_tensor(got):
                got = got.tolist()
                if nulls is not None:
                    got = [None if m else v for v, m in zip(got, nulls.tolist())]
            assert len(got) == len(want), name
            for a, b in zip(got, want):
                if isinstance(b, float) and b is not None and a is not None:
                    assert a == b or (math.isnan(a) and math.isnan(b)), name
                else:
                    assert a == b, (name, a, b)


@pytest.mark.parametrize("codec", ["none", "snappy", "gzip", "zstd"])
@pytest.mark.parametrize("version", ["1.0", "2.0"])
@pytest.mark.parametrize("dictionary", [True, False])
def test_codecs_page_versions_dictionaries(tmp_path, codec, version, dictionary):
    p = str(tmp_path / "t.parquet")
    pq.write_table(pa.table(_table(3000)), p, compression=codec, data_page_version=version, use_dictionary=dictionary,
                   row_group_size=1100, data_page_size=4096)
    _check_against_arrow(p, 3)


@pytest.mark.parametrize("encoding", ["DELTA_BINARY_PACKED", "DELTA_LENGTH_BYTE_ARRAY", "DELTA_BYTE_ARRAY", "BYTE_STREAM_SPLIT", "RLE"])
def test_column_encodings(tmp_path, encoding):
    t = _table(2500, seed=1)
    pick = {"DELTA_BINARY_PACKED": ["i32", "i64", "seq", "opt_i"], "DELTA_LENGTH_BYTE_ARRAY": ["cat", "uniq", "blob", "opt_s"],
            "DELTA_BYTE_ARRAY": ["cat", "uniq", "blob", "opt_s", "fix"], "BYTE_STREAM_SPLIT": ["f32", "f64", "opt", "all_null"],
            "RLE": ["flag"]}[encoding]
    p = str(tmp_path / "e.parquet")
    try:
        pq.write_table(pa.table({k: t[k] for k in pick}), p, use_dictionary=False, column_encoding={k: encoding for k in pick},
                       compression="snappy", data_page_version="2.0", data_page_size=2048)
    except Exception as e:   # an older writer without this encoding for this type
        pytest.skip(str(e))
    _check_against_arrow(p)


def test_whole_file_read_matrix_and_shards(tmp_path):
    from mimir_b200.data import datasets
    p = str(tmp_path / "d.parquet")
    n = 250
    cols = {"f0": torch.randn(n), "f1": torch.randn(n).double(), "label": torch.arange(n) % 3, "name": ["r%d" % i for i in range(n)]}
    parquet.write(p, cols, compression="zstd", row_group_size=100)
    with parquet.File(p) as f:
        assert f.row_groups == 3 and f.schema()["name"].startswith("BYTE_ARRAY")
        got = f.read()
        assert torch.equal(got["f0"], cols["f0"]) and torch.equal(got["f1"], cols["f1"]) and torch.equal(got["label"], cols["label"])
        assert got["name"] == cols["name"]
        X, y = f.matrix(["f0", "f1"], "label", row_group=1)
        assert X.shape == (100, 2) and torch.equal(y, cols["label"][100:200])
        assert sum(len(part["f0"]) for part in f.iter_row_groups(["f0"])) == n
    st = datasets.parquet_shards(p, ["f0", "f1"], "label", batch_size=64)
    assert sum(b.x.shape[0] for b in st) == n


def test_nested_and_unsupported_are_listed_but_refused(tmp_path):
    p = str(tmp_path / "n.parquet")
    pq.write_table(pa.table({"x": pa.array([1, 2, 3], pa.int32()), "l": pa.array([[1], [2, 3], []], pa.list_(pa.int64())),
                             "s": pa.array([{"a": 1.0}, {"a": 2.0}, {"a": None}])}), p)
    f = parquet.File(p)
    info = {c.name: c for c in f.column_info()}
    assert not info["x"].nested and info["l.list.element"].nested and info["s.a"].nested
    assert f.read_column(0, "x")[0].tolist() == [1, 2, 3]
    with pytest.raises(parquet.ErrUnsupported, match="nested"):
        f.read_column(0, "l.list.element")
    assert list(f.read()) == ["x"]                      # the whole-file read takes the readable columns
    p2 = str(tmp_path / "lz4.parquet")
    pq.write_table(pa.table({"x": pa.array(np.arange(100))}), p2, compression="lz4")
    with pytest.raises(parquet.ErrUnsupported, match="LZ4"):
        parquet.File(p2).read_column(0, "x")
    p3 = str(tmp_path / "ts.parquet")
    pq.write_table(pa.table({"t": pa.array([1, 2], pa.timestamp("ns"))}), p3, use_deprecated_int96_timestamps=True)
    with pytest.raises(parquet.ErrUnsupported, match="INT96"):
        parquet.File(p3).read_column(0, "t")


def test_logical_types_are_reported_not_applied(tmp_path):
    import decimal
    p = str(tmp_path / "lt.parquet")
    pq.write_table(pa.table({"d": pa.array([decimal.Decimal("1.25"), decimal.Decimal("-3.50")], pa.decimal128(9, 2)),
                             "day": pa.array([0, 19000], pa.date32()), "ts": pa.array([0, 10**6], pa.timestamp("us")),
                             "u8": pa.array([1, 255], pa.uint8())}), p)
    f = parquet.File(p)
    info = {c.name: c for c in f.column_info()}
    assert info["d"].logical == "DECIMAL" and (info["d"].precision, info["d"].scale) == (9, 2)
    assert info["day"].logical == "DATE" and info["ts"].logical == "TIMESTAMP" and info["u8"].logical == "INTEGER"
    assert f.read_column(0, "day")[0].tolist() == [0, 19000] and f.read_column(0, "ts")[0].tolist() == [0, 10**6]
    assert f.read_column(0, "u8")[0].tolist() == [1, 255]


# ------------------------------------------------------------------ hostile bytes
def _good(tmp_path):
    p = str(tmp_path / "g.parquet")
    pq.write_table(pa.table(_table(400, seed=3)), p, compression="snappy", data_page_version="2.0", row_group_size=150)
    return p, open(p, "rb").read()


def _try_all(path):
    f = parquet.File(path)
    for g in range(f.row_groups):
        for c in f.column_info():
            if not c.nested:
                f.read_column(g, c.name)


def test_truncated_and_garbled_files_fail_with_an_error(tmp_path):
    p, good = _good(tmp_path)
    bad = str(tmp_path / "bad.parquet")
    for cut in (0, 3, 4, 11, 12, len(good) // 2, len(good) - 9, len(good) - 1):
        open(bad, "wb").write(good[:cut])
        with pytest.raises((parquet.ParquetError, OSError)):
            _try_all(bad)
    open(bad, "wb").write(b"PAR1" + good[4:-4] + b"PARE")
    with pytest.raises(parquet.ErrUnsupported, match="encrypted"):
        parquet.File(bad)
    # footer length pointing outside the file
    open(bad, "wb").write(good[:-8] + struct.pack("<I", len(good)) + b"PAR1")
    with pytest.raises(parquet.ErrFormat):
        parquet.File(bad)


def test_random_byte_flips_never_crash(tmp_path):
    p, good = _good(tmp_path)
    bad = str(tmp_path / "flip.parquet")
    rng = np.random.default_rng(11)
    refused = 0
    for trial in range(300):
        b = bytearray(good)
        # footers and page headers are where a flipped byte does the most damage
        lo = len(b) - 600 if trial % 2 else 4
        for _ in range(1 + trial % 4):
            pos = int(rng.integers(lo, len(b) - 8))
            b[pos] = int(rng.integers(0, 256))
        open(bad, "wb").write(bytes(b))
        try:
            _try_all(bad)
        except (parquet.ParquetError, OSError, IndexError, KeyError):
            refused += 1
    assert refused > 30      # and no crash, no hang, no unbounded allocation on the way


def test_hostile_counts_are_refused_before_allocation(tmp_path):
    # a footer that declares 2^40 rows in its only row group: refused, not allocated
    p, good = _good(tmp_path)
    f = parquet.File(p)
    assert f.rows == 400
    # patch the snappy length varint of the first page to claim more than the header says
    bad = str(tmp_path / "h.parquet")
    idx = good.find(b"\x15\x06")          # a page header start (type field, DATA_PAGE_V2 = 3 zigzag 6)
    if idx < 0:
        pytest.skip("page header pattern not found")
    b = bytearray(good)
    b[idx + 3] ^= 0x40                    # disturb the uncompressed size
    open(bad, "wb").write(bytes(b))
    with pytest.raises((parquet.ParquetError, IndexError)):
        _try_all(bad)
