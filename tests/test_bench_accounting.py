"""The arithmetic behind bench.py's roofline keys, on the CPU: compulsory bytes per product, the fraction of the measured
copy bandwidth, and which stages count as in line with the pass."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402

N_IN, N_OUT, PAIRS = 1_200_000, 836_131, 4_427_397
PK = {"hbm_gbs": 6533.8, "bf16_tflops": 1638.1, "source": "measured"}


def test_compulsory_bytes_of_the_products():
    """e*(N_in*Cin + N_out*Cout + K*Cin*Cout) + 4*rows*K with the forward map's rows for fwd / wgrad and the inverse
    map's for dgrad: 458 MB and 498 MB on the default layer in bf16."""
    es, K, cin, cout = 2, bench.K, bench.CIN, bench.COUT
    tensors = es * (N_IN * cin + N_OUT * cout + K * cin * cout)
    for kind, rows in (("conv_fwd", N_OUT), ("conv_wgrad", N_OUT), ("conv_dgrad", N_IN)):
        compulsory, gathered = bench.conv_bytes(kind, N_IN, N_OUT, PAIRS, es)
        assert compulsory == tensors + 4 * rows * K
        assert gathered > compulsory                       # the gathers fetch an input row once per pair
    assert round(bench.conv_bytes("conv_fwd", N_IN, N_OUT, PAIRS, es)[0] / 1e6) == 458
    assert round(bench.conv_bytes("conv_dgrad", N_IN, N_OUT, PAIRS, es)[0] / 1e6) == 498


def test_fraction_is_bytes_over_time_over_the_measured_peak():
    per_stage = {"conv_wgrad": {"ms_per_pass": 0.445, "launches_per_pass": 2},
                 "conv_wgrad_presort": {"ms_per_pass": 0.1, "launches_per_pass": 1},
                 "map_plan": {"ms_per_pass": 0.17, "launches_per_pass": 11},
                 "out_coords": {"ms_per_pass": 0.157, "launches_per_pass": 10}}
    roofs = bench.stage_rooflines(per_stage, N_IN, N_OUT, PAIRS, PK, torch.bfloat16, 49_500, 34_600)
    w = roofs["conv_wgrad"]
    assert w["bound"] == "hbm"                             # 158 flop/B x 6.5 TB/s is below the tensor peak
    assert w["frac"] == pytest.approx(w["algorithmic_bytes"] / 0.445e-3 / 1e9 / PK["hbm_gbs"])
    assert w["frac"] == pytest.approx(0.1577, abs=2e-4)
    assert w["tensor_frac"] == pytest.approx(2.0 * PAIRS * bench.CIN * bench.COUT / 0.445e-3 / 1e12 / PK["bf16_tflops"])
    # one 128-row x 128-byte slot per (tile, offset) step against the measured row-gather rate
    assert w["gather_slot_bytes"] == 49_500 * 128 * 128
    assert w["gather_frac"] == pytest.approx(w["gather_slot_bytes"] / 0.445e-3 / 1e9 / bench.GATHER_CEILING_GBS)
    # the copy of dY into tile order: read and written once, plus the row order
    assert roofs["conv_wgrad_presort"]["algorithmic_bytes"] == 2 * N_OUT * bench.COUT * 2 + 4 * N_OUT
    assert roofs["map_plan"]["algorithmic_bytes"] == 8 * bench.K * N_OUT
    assert roofs["out_coords"]["algorithmic_bytes"] == pytest.approx(N_IN * (16 + 12 * 27 / 8.0) + 16 * N_OUT)


def test_fp32_products_are_held_to_half_the_bf16_tensor_peak():
    per_stage = {"conv_fwd": {"ms_per_pass": 0.6, "launches_per_pass": 1}}
    r = bench.stage_rooflines(per_stage, N_IN, N_OUT, PAIRS, PK, torch.float32)["conv_fwd"]
    assert r["algorithmic_bytes"] == bench.conv_bytes("conv_fwd", N_IN, N_OUT, PAIRS, 4)[0]
    assert r["tensor_frac"] == pytest.approx(r["tflops"] / (PK["bf16_tflops"] * 0.5))
