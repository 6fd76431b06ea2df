import torch

import gpu_mode_kernels_b200 as pkg
from gpu_mode_kernels_b200 import traffic


def test_pair_counts_small():
    idx = [torch.tensor([[0, 1], [2, 3]], dtype=torch.int32), torch.tensor([[0, 2], [1, 0]], dtype=torch.int32)]
    pairs, rows = traffic.pair_counts(idx, 4, 2)  # experts 0,1 on rank 0; 2,3 on rank 1
    assert pairs.tolist() == [[2, 2], [3, 1]]
    assert rows.tolist() == [[1, 1], [2, 1]]
    s = traffic.summarize(idx, 4, 2, 64)
    assert s["busiest_rows"] == 3 and s["busiest_rows_dedup"] == 2
    assert s["algorithmic_bytes"] == 3 * (128 + 128)
    assert s["total_pairs"] == 8 and s["local_pairs"] == 3


def test_headline_workload_floor_matches_published_analysis():
    """c4 at world size 8: ~1.8k rows on the busiest rank, ~58 us at 900 GB/s for dispatch+combine."""
    idx = [pkg.workload_input("c4", r, 8)[1].indices for r in range(8)]
    s = traffic.summarize(idx, 256, 8, 7168)
    assert 1750 <= s["busiest_rows"] <= 1900
    assert 55.0 <= s["t_roof_us_nominal"] <= 61.0
    assert s["busiest_rows_dedup"] < 0.72 * s["busiest_rows"]


def test_single_rank_hbm_bytes():
    b = traffic.hbm_bytes_single_rank(256, 8, 7168)
    assert b["recv_expert"] == 2 * 2048 * 14336
    assert b["dispatch_send"] == (256 + 2048) * 14336


def test_wire_bytes_follow_payload_and_combine_mode():
    """Algorithmic bytes never change; the wire carries one row per (token, rank) where the payload
    (dispatch) or the expert-side reduction (combine) deduplicates."""
    idx = [pkg.workload_input("c4", r, 8)[1].indices for r in range(8)]
    H = 7168
    direct = traffic.summarize(idx, 256, 8, H, "direct", "pull")
    dedup_pull = traffic.summarize(idx, 256, 8, H, "dedup", "pull")
    dedup_push = traffic.summarize(idx, 256, 8, H, "dedup", "push")
    fp8_push = traffic.summarize(idx, 256, 8, H, "fp8", "push")
    assert direct["algorithmic_bytes"] == dedup_pull["algorithmic_bytes"] == dedup_push["algorithmic_bytes"]
    assert direct["wire_bytes"] == direct["algorithmic_bytes"]
    b, bd = direct["busiest_rows"], direct["busiest_rows_dedup"]
    assert dedup_pull["wire_bytes"] == (bd + b) * 2 * H
    assert dedup_push["wire_bytes"] == 2 * bd * 2 * H
    assert fp8_push["wire_bytes"] == bd * (H + 4 * (H // 128)) + bd * 2 * H
    assert dedup_push["t_wire_us_nominal"] < dedup_pull["t_wire_us_nominal"] < direct["t_roof_us_nominal"]
