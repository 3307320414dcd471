"""Seeded generators: shards regenerate the same values; encodings are what they claim."""
import numpy as np

from rocwmma_b200 import synth


def test_row_shards_regenerate_identically():
    full = synth.rows(9, 1, synth.F16, 0, 1024, 64)
    for world in (2, 4, 8):
        per = 1024 // world
        parts = [synth.rows(9, 1, synth.F16, r * per, per, 64) for r in range(world)]
        assert np.array_equal(np.concatenate(parts).view(np.uint16), full.view(np.uint16))


def test_distributions_and_encodings():
    u = synth.rows(1, 1, synth.F32, 0, 256, 256)
    assert u.min() >= -1 and u.max() <= 1 and abs(u.mean()) < 0.02
    x = synth.rows(1, 2, synth.XF32, 0, 128, 64)
    assert not (x.view(np.uint32) & 0x1FFF).any()
    i8 = synth.rows(1, 3, synth.I8, 0, 256, 256, dist="int8")
    assert i8.min() == -128 and i8.max() == 127
    n = synth.rows(1, 4, synth.F16, 0, 256, 256, dist="normal").astype(np.float32)
    assert abs(n.std() - 1) < 0.02
    p = synth.rows(1, 5, synth.F16, 0, 128, 8, dist="pattern").astype(np.float32)
    assert set(np.unique(np.abs(p))) <= {0, 1, 2, 3, 4}
    e = synth.rows(1, 6, synth.E4M3, 0, 128, 64, dist="normal", scale=100.0)
    assert np.abs(synth.e4m3_bits_to_f32(e)).max() <= 448


def test_benchmark_table_rows_match_the_reference_header():
    """bench_configs.py --csv writes rocWMMA's result table: one value per header column."""
    import bench_configs as B
    cols = [c.strip() for c in B.CSV_HEADER.split(",")]
    assert cols[:5] == ["TBlkX", "TBlkY", "BlkM", "BlkN", "BlkK"] and cols[-1] == "Result"
    for simple, in_t, out_t in [(True, B.F16, B.F32), (False, B.E5M2, B.BF16),
                                (False, B.F64, B.F64), (False, B.I8, B.I32)]:
        r = {"ms": 0.5, "value": 100.0, "roofline": {"frac": 0.25},
             "gemm": {"in_t": in_t, "out_t": out_t, "size": 1024, "alpha": 1.0, "beta": 0.0,
                      "simple": simple}}
        row = [c.strip() for c in B.csv_row(r).split(",")]
        assert len(row) == len(cols)
        assert row[cols.index("Result")] == "BENCH"
        assert row[cols.index("Efficiency(%)")] == "25.00"
        assert B.csv_row(dict(r, parity=True)).endswith("PASSED")
        assert B.csv_row(dict(r, parity=False)).endswith("FAILED")
    assert "bf8_bf16_f32" in B.csv_row({"ms": 1, "value": 1, "roofline": {"frac": 1}, "gemm": {
        "in_t": B.E5M2, "out_t": B.BF16, "size": 64, "alpha": 1, "beta": 0, "simple": False}})


def test_threaded_generation_gives_the_same_values():
    a = synth.rows(7, 1, synth.F16, 256, 1000, 96, threads=1)
    b = synth.rows(7, 1, synth.F16, 256, 1000, 96, threads=6)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
