"""Launch configurations that won on 8 x B200 (NVLink 5 / NVSwitch), keyed by op and problem: what ``autotune=True``
(the contextual autotuner of ``tools/autotuner.py``) chose for the benchmark shapes, kept here so that the default path
starts from measured values instead of re-tuning in every process.  An op looks its shape up with :func:`lookup`; a
shape that is not listed falls back to the op's analytical model (e.g. ``pick_comm_ctas``).

How an entry gets here: run the op once with ``autotune=True`` on the target box (every rank, same arguments), read the
``best`` line for the key in ``./.autotune_logs/rank-0.log`` and copy it below.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

# (op, world, rows per rank, N local, K) -> knobs
_TABLE: Dict[Tuple[str, int, int, int, int], Dict] = {
    # AG -> GEMM, M = 8192 tokens, K = 8192, N = 28672 / W (the MLP up-projection of the headline benchmark).
    # Two ranks: nothing to replicate, four unicast comm CTAs keep the 64 MB shard ahead of the GEMM (no flag stalls).
    ("ag_gemm", 2, 4096, 14336, 8192): {"use_multimem": False, "n_comm_ctas": 4},
    # Four and eight ranks: the NVLS ring push with four comm CTAs (every byte leaves the GPU once); at eight ranks ten
    # unicast comm CTAs starved the GEMM for a third of its time and twenty cost a whole wave of tiles.
    ("ag_gemm", 4, 2048, 7168, 8192): {"use_multimem": True, "n_comm_ctas": 4},
    ("ag_gemm", 8, 1024, 3584, 8192): {"use_multimem": True, "n_comm_ctas": 4},
    # Decode GEMM, cluster form ("skinny_gemm", 1, token pad, N, K): CTA tile width in 128-column blocks and CTAs per
    # tile, where `benchmarks/tune_skinny.py` found a pair at least 3 % faster than the launcher's cost model on a
    # 148-SM B200 (Qwen3-32B per-rank shapes; microseconds: winner / model / cuBLAS).
    ("skinny_gemm", 1, 16, 6400, 5120): {"cluster_nt": 2, "cluster_s": 4},    # TP8 gate_up   15.5 / 16.0 / 14.7
    ("skinny_gemm", 1, 32, 6400, 5120): {"cluster_nt": 2, "cluster_s": 4},    #               16.8 / 17.5 / 15.4
    ("skinny_gemm", 1, 16, 5120, 3200): {"cluster_nt": 2, "cluster_s": 6},    # TP8 down      11.1 / 11.7 / 10.1
    ("skinny_gemm", 1, 16, 2560, 5120): {"cluster_nt": 2, "cluster_s": 8},    # TP4 qkv       10.3 / 10.7 / 10.3
    ("skinny_gemm", 1, 16, 5120, 2048): {"cluster_nt": 2, "cluster_s": 4},    # TP4 o_proj     9.3 /  9.8 /  7.9
    ("skinny_gemm", 1, 16, 5120, 5120): {"cluster_nt": 2, "cluster_s": 6},    # TP2 qkv       13.9 / 14.7 / 13.6
}


_USER_TABLE: Optional[Dict[Tuple[str, int, int, int, int], Dict]] = None


def _user_table() -> Dict[Tuple[str, int, int, int, int], Dict]:
    """Entries from the JSON file named by ``TDB200_TUNED_CONFIGS`` (read once per process): a list of
    ``{"op", "world", "rows", "n", "k", "config": {...}}`` records, as ``benchmarks/tune_skinny.py --json-out`` writes
    them.  They come before the built-in table, so a box can carry its own winners without a source change."""
    global _USER_TABLE
    if _USER_TABLE is None:
        import json
        import os

        table: Dict[Tuple[str, int, int, int, int], Dict] = {}
        path = os.environ.get("TDB200_TUNED_CONFIGS", "")
        if path:
            with open(path) as f:
                for rec in json.load(f):
                    key = (str(rec["op"]), int(rec["world"]), int(rec["rows"]), int(rec["n"]), int(rec["k"]))
                    table[key] = dict(rec["config"])
        _USER_TABLE = table
    return _USER_TABLE


def lookup_user(op: str, world: int, rows_per_rank: int, n_local: int, k: int) -> Optional[Dict]:
    """The entry of the user's table only (measured on the box it runs on)."""
    return _user_table().get((op, int(world), int(rows_per_rank), int(n_local), int(k)))


def lookup(op: str, world: int, rows_per_rank: int, n_local: int, k: int) -> Optional[Dict]:
    key = (op, int(world), int(rows_per_rank), int(n_local), int(k))
    user = _user_table()
    return user[key] if key in user else _TABLE.get(key)
