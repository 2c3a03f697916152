"""Cross-rank reading of flight-recorder dumps: where did the ranks part ways?

    python -m torchcomms_b200.hooks.fr_analyze /tmp/b200c_fr_trace_*          # one dump file per rank
    report = analyze([json.load(open(p)) for p in paths])

For every communicator the dumps are lined up by collective sequence number and the report names

* the first sequence number at which the ranks issued **different operations or sizes** (a desynchronised
  program: one rank called ``all_gather`` where the others called ``all_reduce``, or with another shape);
* operations some ranks **never issued** (a rank that stopped calling: the others hang in that collective);
* operations issued everywhere but **not completed** on some ranks, with the ranks that lag;
* per rank, the last enqueued / started / completed sequence numbers.

This is the hang triage the recorder exists for; the dumps come from ``FlightRecorderHook.dump_file`` (written
by the abort hook on a timeout).  Parity: the reference feeds the same c10d-format dumps to an analyzer service
(comms/analyzer/if, Thrift interface only); PyTorch's ``fr_trace`` script reads the format too.
"""
from __future__ import annotations

import json
import sys
from typing import Any, Dict, List, Optional, Sequence


def _signature(e: Dict[str, Any]) -> tuple:
    return (e.get("profiling_name"), json.dumps(e.get("input_sizes")), json.dumps(e.get("output_sizes")),
            json.dumps(e.get("input_dtypes")))


def analyze(dumps: Sequence[Dict[str, Any]]) -> Dict[str, Any]:
    """``dumps``: one parsed dump per rank (any order). Returns a report dict, one entry per communicator."""
    by_comm: Dict[str, Dict[int, Dict[int, Dict[str, Any]]]] = {}
    status: Dict[str, Dict[int, Dict[str, Any]]] = {}
    for d in dumps:
        rank = int(d.get("rank", 0))
        for name, st in (d.get("pg_status") or {}).items():
            status.setdefault(name, {})[rank] = st
        for e in d.get("entries", []):
            if e.get("is_p2p"):
                continue                                    # point-to-point sequences are pairwise, not collective
            comm = e["process_group"][0]
            by_comm.setdefault(comm, {}).setdefault(rank, {})[int(e["collective_seq_id"])] = e
    report: Dict[str, Any] = {}
    for comm, per_rank in by_comm.items():
        ranks = sorted(per_rank)
        # only sequence numbers every rank's ring still holds can be compared for content
        first_kept = max(min(seqs) for seqs in per_rank.values())
        last_any = max(max(seqs) for seqs in per_rank.values())
        mismatch: Optional[Dict[str, Any]] = None
        missing: List[Dict[str, Any]] = []
        incomplete: List[Dict[str, Any]] = []
        for seq in range(first_kept, last_any + 1):
            have = {r: per_rank[r][seq] for r in ranks if seq in per_rank[r]}
            absent = [r for r in ranks if r not in have]
            if absent:
                missing.append({"seq": seq, "op": next(iter(have.values()))["profiling_name"], "ranks_without": absent})
                continue
            sigs = {r: _signature(e) for r, e in have.items()}
            if mismatch is None and len(set(sigs.values())) > 1:
                mismatch = {"seq": seq, "by_rank": {r: {"op": s[0], "input_sizes": json.loads(s[1])} for r, s in sigs.items()}}
            lagging = [r for r, e in have.items() if e.get("state") != "completed"]
            if lagging:
                incomplete.append({"seq": seq, "op": have[ranks[0]]["profiling_name"],
                                   "states": {r: have[r].get("state") for r in lagging}})
        report[comm] = {
            "ranks": ranks,
            "first_mismatch": mismatch,
            "never_issued": missing,
            "not_completed": incomplete,
            "progress": {r: status.get(comm, {}).get(r, {}) for r in ranks},
        }
    return report


def format_report(report: Dict[str, Any]) -> str:
    lines: List[str] = []
    for comm, r in report.items():
        lines.append(f"communicator '{comm}' (ranks {r['ranks']})")
        if r["first_mismatch"]:
            m = r["first_mismatch"]
            lines.append(f"  ranks disagree at collective {m['seq']}:")
            for rank, what in m["by_rank"].items():
                lines.append(f"    rank {rank}: {what['op']} {what['input_sizes']}")
        for m in r["never_issued"][:5]:
            lines.append(f"  collective {m['seq']} ({m['op']}) was never issued by ranks {m['ranks_without']}")
        for m in r["not_completed"][:5]:
            lines.append(f"  collective {m['seq']} ({m['op']}) not completed on {m['states']}")
        if not (r["first_mismatch"] or r["never_issued"] or r["not_completed"]):
            lines.append("  all ranks issued and completed the same collectives")
        for rank, st in r["progress"].items():
            if st:
                lines.append(f"  rank {rank}: enqueued {st.get('last_enqueued_collective')}, started "
                             f"{st.get('last_started_collective')}, completed {st.get('last_completed_collective')}")
    return "\n".join(lines)


def main(argv: Optional[List[str]] = None) -> int:
    paths = (argv if argv is not None else sys.argv[1:])
    if not paths:
        print(__doc__)
        return 2
    dumps = []
    for p in paths:
        with open(p) as f:
            dumps.append(json.load(f))
    print(format_report(analyze(dumps)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
