"""Run the REFERENCE project's v4 / v5 per-layer planners on the seeded layers of planner_cases.py
and store their decisions in planner_decisions.json.

    python tests/golden/make_planner_golden.py --reference /path/to/ai_accel_studio

The reference is imported read-only and runs on the CPU, where its timed speed gate reports
"not measured" (None) and every quality-passing candidate is accepted; what the fixture pins is
therefore the candidate search and its tie-breaking.  tests/test_planner_cpu.py runs this
package's planner on the same layers and compares.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from ai_accel_lab.optimize.planner_v4 import decide_linear_v4
    from ai_accel_lab.optimize.planner_v5 import decide_linear_v5
    import planner_cases as pc

    out = {}
    for name in pc.CASES:
        layer, x, kw = pc.make_case(name)
        kw4 = {k: v for k, v in kw.items() if k in ("group_sizes", "outliers", "residual_ranks", "nmse_limit", "cosine_limit")}
        out[name] = dict(v4=decide_linear_v4(name, layer, x, **kw4).to_dict(), v5=decide_linear_v5(name, layer, x, **kw).to_dict())
        print(name, out[name]["v5"])
    (HERE / "planner_decisions.json").write_text(json.dumps(out, indent=1, sort_keys=True))


if __name__ == "__main__":
    main()
