"""Writes the golden fixtures of tests/test_oracle.py::test_golden_fixture.

The reference project (ernie-research/ERNIE-Evolve-Results) ships no vectors,
tests or importable Python for the routing/dispatch path, so the fixtures are
outputs of this repository's CPU oracle on the seeded workloads: small index
and weight arrays verbatim, large row buffers as SHA-256 digests.

    python tests/golden/make_golden.py
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path[:0] = [str(ROOT), str(ROOT / "ernie-evolve-results_b200"), str(HERE.parent)]

from moe_rd import workloads  # noqa: E402
import _util  # noqa: E402

CASES = {"c1": ("c1", None, None), "c2_small": ("c2", 640, 1024), "c3_small": ("c3", 1500, 512),
         "c4_small": ("c4", 333, 1024)}


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


for name, (wl, T, H) in CASES.items():
    t, kw = workloads.make(wl, T=T, H=H)
    r = _util.run_oracle(t, kw)
    meta = {"workload": wl, "T": T, "H": H, "x_sha256": digest(_util.bf16_bits(t["x"])),
            "permuted_sha256": digest(r["permuted"]),
            "scales_sha256": digest(r["scales"]) if r["scales"] is not None else None,
            "kept_rows": int(r["offsets"][-1]), "dropped": int(r["drop_mask"].sum())}
    (HERE / f"{name}.json").write_text(json.dumps(meta, indent=1) + "\n")
    np.savez_compressed(HERE / f"{name}.npz", expert_ids=r["expert_ids"], offsets=r["offsets"],
                        inverse_perm=r["inverse_perm"], combine_weights=r["combine_weights"])
    print(name, meta["kept_rows"], meta["dropped"])
