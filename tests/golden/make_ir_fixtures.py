"""Writes tests/golden/ir/call_<name>.json: lowered call IR ("lowered-ir-v3", decode mode) produced by the reference's OWN lowering
pipeline (version/v7/scripts/build_ir_v7.py, run as it lies in the reference checkout) for the small models of tests/ir_cases.py.

    CK_REFERENCE_DIR=/path/to/C-Kernel-Engine python tests/golden/make_ir_fixtures.py

For each case a BUMPWGT5 file and its map are written to a scratch folder (tests/bump_file.py), a manifest JSON with the keys the
builder reads is put beside them, and the builder is invoked with --call-output.  Nothing of the output is edited.  The IR depends
only on shapes, formats and the template, not on weight values, so tests regenerate the weights from their seed."""
from __future__ import annotations

import json
import os
import pathlib
import shutil
import subprocess
import sys
import tempfile

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import bump_file          # noqa: E402
import ir_cases           # noqa: E402
import step_oracle as so  # noqa: E402


def main():
    ref = pathlib.Path(os.environ.get("CK_REFERENCE_DIR", HERE.parents[2] / "reference"))
    builder = ref / "version" / "v7" / "scripts" / "build_ir_v7.py"
    if not builder.exists():
        sys.exit(f"{builder} not found: set CK_REFERENCE_DIR to a checkout of the reference")
    out_dir = HERE / "ir"
    out_dir.mkdir(exist_ok=True)
    for name, (arch, cfg, seed) in ir_cases.CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            tmp = pathlib.Path(tmp)
            cpu = so.CpuModel(cfg, seed=seed)
            entries = bump_file.write_bump(tmp / "weights.bump", tmp / "weights_manifest.map", cpu)
            (tmp / "weights_manifest.json").write_text(json.dumps(ir_cases.manifest_dict(arch, cfg, entries), indent=1))
            cmd = [sys.executable, str(builder), "--manifest", str(tmp / "weights_manifest.json"), "--mode", "decode", "--output", str(tmp / "ir1.json"),
                   "--layout-output", str(tmp / "layout.json"), "--lowered-output", str(tmp / "lowered.json"), "--call-output", str(tmp / "call.json")]
            r = subprocess.run(cmd, capture_output=True, text=True, cwd=tmp)
            if r.returncode or not (tmp / "call.json").exists():
                sys.exit(f"{name}: the reference's IR builder failed\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}")
            shutil.copyfile(tmp / "call.json", out_dir / f"call_{name}.json")
            doc = json.loads((out_dir / f"call_{name}.json").read_text())
            print(f"{name}: {len(doc['operations'])} ops, {sorted(set(op['function'] for op in doc['operations']))}")


if __name__ == "__main__":
    main()
