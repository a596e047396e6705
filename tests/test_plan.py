"""CPU: the tile-plan chooser (host-only code of the library) and its overrides."""
import ctypes
import os
import subprocess
import sys

import open64_b200 as o

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def model(kind, M, N, K, swiglu=0, sms=148, **pin):
    p = o.Plan()
    pp = None
    if pin:
        pp = o.Plan()
        for k, v in pin.items():
            setattr(pp, k, v)
        pp = ctypes.byref(pp)
    rc = o.lib().o64_plan_model(kind, swiglu, M, N, K, sms, pp, ctypes.byref(p))
    assert rc == 0
    return p.as_dict()


def test_headline_shapes(built):
    p = model(o.KIND_BF16, 8192, 8192, 8192)
    assert (p["tile_n"], p["tile_k"]) == (256, 64) and p["stages"] in (4, 6)
    # the headline shape takes the widest form: a CTA pair per 512 x 256 tile
    assert (p["cta_group"], p["tile_m"]) == (2, 512)
    assert (p["mma_n"], p["mma_k"]) == (256, 16)
    assert p["num_ctas"] == 148 and (p["cta_group"], p["tile_m"]) in ((1, 128), (2, 256), (2, 512))
    assert 0.4 < p["predicted_ms"] < 1.5
    for kind in (o.KIND_FP8, o.KIND_S8):
        p = model(kind, 4096, 8192, 8192)
        assert p["tile_k"] == 128 and p["mma_k"] == 32
    # shared-memory ring fits: stages * (A + B bytes one CTA stages per K block) <= 227 KB
    for cg, tm in ((1, 128), (2, 256), (2, 512)):
        for tn in (128, 256):
            if tm == 512 and tn == 128:
                continue
            p = model(o.KIND_BF16, 4096, 4096, 4096, tile_n=tn, cta_group=cg, tile_m=tm)
            assert (p["tile_n"], p["cta_group"], p["tile_m"]) == (tn, cg, tm)
            assert p["stages"] * (tm // cg + tn // cg) * 128 + 16384 <= 227 * 1024


def test_group_m_makes_a_near_square_wave(built):
    p = model(o.KIND_BF16, 8192, 8192, 8192, cta_group=1)
    g = p["group_m"]
    cols = 148 / g
    assert g in (8, 16)
    assert g * 128 + cols * 256 <= 8 * 128 + (148 / 8) * 256


def test_pins_and_rejections(built):
    p = model(o.KIND_BF16, 8192, 8192, 8192, tile_n=128, group_m=4, num_ctas=64, raster=1, cta_group=1)
    assert (p["tile_n"], p["group_m"], p["num_ctas"], p["raster"], p["stages"]) == (128, 4, 64, 1, 6)
    pl = o.Plan()
    assert o.lib().o64_plan_model(o.KIND_F32, 0, 8, 8, 8, 148, None, ctypes.byref(pl)) == o.ERR_RANK
    assert o.lib().o64_plan_model(o.KIND_FP8, 1, 8, 8, 8, 148, None, ctypes.byref(pl)) == o.ERR_DTYPE
    assert o.lib().o64_plan_model(o.KIND_BF16, 0, 0, 8, 8, 148, None, ctypes.byref(pl)) == o.ERR_RANK


def test_few_rows_of_a_take_the_cluster_split_kernel(built):
    for kind, eb in ((o.KIND_BF16, 2), (o.KIND_FP8, 1), (o.KIND_S8, 1)):
        for M, rows, cols, stages in ((1, 16, 256, 6), (16, 16, 256, 6), (17, 32, 256, 5), (64, 64, 256, 5),
                                      (100, 128, 128, 6), (128, 128, 128, 6)):
            p = model(kind, M, 8192, 8192)
            # 32 tiles of 256 columns, each split over a cluster of 4 CTAs: 128 of the 148 SMs; more
            # than 64 rows: 64 tiles of 128 columns on clusters of 2 (a third of the partial sums to exchange)
            assert p["split_k"] == (-4 if cols == 256 else -2) and p["num_ctas"] == 128
            assert (p["tile_m"], p["tile_n"], p["cta_group"]) == (rows, cols, 1)
            assert p["stages"] == stages and p["stages"] * (cols + rows) * 128 + 16384 + 1024 + 256 <= 227 * 1024
            # bound by HBM: the weight once at about 6.5 TB/s, plus launch and tail
            assert 8192 * 8192 * eb / 6.5e9 < p["predicted_ms"] < 2.5 * 8192 * 8192 * eb / 6.5e9
    assert model(o.KIND_BF16, 16, 28672, 4096)["split_k"] == -1         # 112 tiles: one CTA each
    assert model(o.KIND_BF16, 16, 2048, 8192)["split_k"] == -8          # 8 tiles: clusters of 8
    p = model(o.KIND_BF16, 16, 4096, 8192)      # 16 tiles of 256 columns would use 64 SMs: 32 of 128 columns
    assert (p["tile_n"], p["split_k"], p["num_ctas"]) == (128, -4, 128)
    assert model(o.KIND_BF16, 16, 8192, 8192, split_k=-8, tile_n=128)["split_k"] == -4   # a CTA owns 32 columns at least
    assert model(o.KIND_BF16, 16, 65536, 128, split_k=-1)["split_k"] == -1
    assert model(o.KIND_BF16, 16, 8192, 8192, split_k=-2)["split_k"] == -2
    assert model(o.KIND_BF16, 129, 8192, 8192)["split_k"] >= 1          # more rows: the tile kernels
    assert model(o.KIND_BF16, 16, 256, 512)["split_k"] >= 1            # a weight that small is not worth it
    assert model(o.KIND_BF16, 16, 8192, 8192, swiglu=1)["split_k"] >= 1
    assert model(o.KIND_BF16, 16, 8192, 8192, split_k=1)["split_k"] == 1
    assert model(o.KIND_BF16, 16, 8192, 8192, cta_group=2)["split_k"] >= 1
    assert model(o.KIND_BF16, 16, 256, 512, split_k=-1)["split_k"] == -8          # asked for: 1 tile, 8 K blocks


def test_env_override_and_trace(built):
    code = ("import ctypes, open64_b200 as o; p=o.Plan();"
            "o.lib().o64_plan_model(1,0,4096,4096,4096,148,None,ctypes.byref(p));"
            "print(p.tile_n,p.group_m,p.num_ctas,p.raster)")
    env = dict(os.environ, O64_LNO="blocking_size=128x128x64:group_m=2:num_ctas=100:raster=1",
               O64_TRACE="plan", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == ["128", "2", "100", "1"]
    assert "[o64 plan" in r.stderr and "tile 128x128x64" in r.stderr
