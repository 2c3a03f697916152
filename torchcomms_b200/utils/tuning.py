"""Offline tuning: turns sweep results into an algorithm table and cross-over sizes.

    torchrun --nproc-per-node 8 benchmarks/collective_perf.py --algos kernel,nccl --json sweep.json
    python -m torchcomms_b200.utils.tuning sweep.json [--emit tuner.txt] [--margin 0.05]   # also reads bench.py --sweep-json files

``--emit`` writes the cross-over table as a tuner file (lines of ``<operation> <largest bytes | inf> <kernel |
nccl>``) that the CUDA backend loads through the hint ``tuner_file`` / ``B200COMMS_TUNER_FILE`` and consults before
its built-in choices; every rank must load the same file.

``best_config(rows)`` maps ``(op, dtype, bytes)`` to the fastest arm;
``crossovers(rows)`` compresses that into byte ranges per operation, the form
in which the CUDA backend's ``route()`` table is written; ``hint_sweep`` helps
comparing sweeps run with different ``--hints`` (chunking, grid size).

Parity: comms/tuning (``comm_tuning`` sweep engine emitting {Key: Config} maps).
"""
from __future__ import annotations

import json
import sys
from typing import Any, Dict, Iterable, List, Tuple

Key = Tuple[str, str, int]


def _normalised(r: Dict[str, Any]) -> Dict[str, Any]:
    """Rows of ``benchmarks/collective_perf.py`` carry ``algo`` / ``us``; rows of the sweep in ``bench.py``
    (``--sweep-json``) carry ``arm`` (``own`` = this framework's kernels) / ``avg_us``."""
    if "algo" in r and "us" in r:
        return r
    arm = r.get("algo", r.get("arm"))
    return {**r, "algo": "kernel" if arm == "own" else arm, "us": r.get("us", r.get("avg_us"))}


def best_config(rows: Iterable[Dict[str, Any]], margin: float = 0.0) -> Dict[Key, Dict[str, Any]]:
    """Fastest arm per (op, dtype, bytes). With ``margin`` (say 0.05) the ``nccl`` arm has to be faster than the
    best other arm by that fraction to be chosen: differences inside the noise of a short sweep should not make
    the route flip from size to size."""
    by_key: Dict[Key, List[Dict[str, Any]]] = {}
    for r in map(_normalised, rows):
        by_key.setdefault((r["op"], r.get("dtype", ""), int(r["bytes"])), []).append(r)
    best: Dict[Key, Dict[str, Any]] = {}
    for key, arms in by_key.items():
        own = [a for a in arms if a["algo"] != "nccl"]
        ref = [a for a in arms if a["algo"] == "nccl"]
        pick = min(arms, key=lambda a: a["us"])
        if margin > 0.0 and own and ref:
            o, n = min(own, key=lambda a: a["us"]), min(ref, key=lambda a: a["us"])
            pick = n if n["us"] < o["us"] * (1.0 - margin) else o
        best[key] = {"algo": pick["algo"], "us": pick["us"]}
    return best


def crossovers(rows: Iterable[Dict[str, Any]], margin: float = 0.0) -> Dict[Tuple[str, str], List[Tuple[int, int, str]]]:
    """Per (op, dtype): maximal runs of consecutive sizes won by the same arm, as (first_bytes, last_bytes, algo)."""
    best = best_config(rows, margin)
    out: Dict[Tuple[str, str], List[Tuple[int, int, str]]] = {}
    for (op, dt, b) in sorted(best, key=lambda k: (k[0], k[1], k[2])):
        algo = best[(op, dt, b)]["algo"]
        runs = out.setdefault((op, dt), [])
        if runs and runs[-1][2] == algo:
            runs[-1] = (runs[-1][0], b, algo)
        else:
            runs.append((b, b, algo))
    return out


def hint_sweep(named_rows: Dict[str, Iterable[Dict[str, Any]]], arm: str = "kernel") -> Dict[Key, Dict[str, Any]]:
    """Several sweeps of the same arm under different hints -> the best hint set per (op, dtype, bytes)."""
    best: Dict[Key, Dict[str, Any]] = {}
    for name, rows in named_rows.items():
        for r in rows:
            if r["algo"] not in (arm, "auto"):
                continue
            key = (r["op"], r.get("dtype", ""), int(r["bytes"]))
            if key not in best or r["us"] < best[key]["us"]:
                best[key] = {"hints": name, "us": r["us"]}
    return best


def tuner_file_lines(rows: Iterable[Dict[str, Any]], dtype: str = "bf16", margin: float = 0.0) -> List[str]:
    """The cross-overs of one dtype as tuner-file lines; arms other than ``nccl`` count as ``kernel``."""
    lines = ["# operation  largest message (bytes)  algorithm"]
    for (op, dt), runs in sorted(crossovers(rows, margin).items()):
        if dt != dtype:
            continue
        merged: List[Tuple[int, str]] = []
        for _, last, algo in runs:
            algo = "nccl" if algo == "nccl" else "kernel"
            if merged and merged[-1][1] == algo:
                merged[-1] = (last, algo)
            else:
                merged.append((last, algo))
        for i, (last, algo) in enumerate(merged):
            lines.append(f"{op} {'inf' if i == len(merged) - 1 else last} {algo}")
    return lines


def main(argv: List[str]) -> int:
    args = list(argv[1:])
    emit = None
    margin = 0.0
    if "--emit" in args:
        i = args.index("--emit")
        emit = args[i + 1]
        del args[i:i + 2]
    if "--margin" in args:
        i = args.index("--margin")
        margin = float(args[i + 1])
        del args[i:i + 2]
    if not args:
        print(__doc__)
        return 2
    rows: List[Dict[str, Any]] = []
    for path in args:
        rows += json.load(open(path))
    for (op, dt), runs in crossovers(rows, margin).items():
        print(f"{op} {dt}: " + ", ".join(f"[{a}..{b}] -> {algo}" for a, b, algo in runs))
    if emit:
        with open(emit, "w") as f:
            f.write("\n".join(tuner_file_lines(rows, margin=margin)) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main(sys.argv))
