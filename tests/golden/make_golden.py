"""Generate the golden fixtures in this directory from the REAL reference.

Run in the authoring container, where the reference checkout is importable:

    PYTHONPATH=/path/to/FuseML python tests/golden/make_golden.py

The reference is Python and cannot travel to a GPU machine, so its outputs are
committed here as small fixtures:

* ``numeric_<cfg>.npz`` — for each benchmark configuration (cfg1 at full size, the
  others scaled down, same seeded generators as ``oracle/configs.py``): the output
  of ``torch.compile(module, backend=fuseml.FuseMLCompiler())`` on CPU, the
  compiler's ``fusion_applied`` / ``fusion_strategy``, and a SHA-256 of the inputs.
  cfg3 selects a Triton group and cannot execute without a GPU driver
  ("0 active drivers"); its fixture holds the eager module's output instead — the
  result the reference's own correctness gate compares against
  (benchmarks/bench_mlp_block.py:453-485) — and says so in ``how``.
* ``structure.json`` — what the reference's discovery pass
  (``FuseMLFusionPass._find_fusion_groups``) finds on the ATen graphs of the same
  modules: per group the op signature, the ordered kernel inputs and the output
  shape.  The new front end must find the same groups with default settings.
"""
from __future__ import annotations

import hashlib
import json
import logging
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import configs  # noqa: E402


def _sha(tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(np.ascontiguousarray(t.detach().numpy()).tobytes())
    return h.hexdigest()


def main() -> None:
    logging.disable(logging.INFO)
    import fuseml  # the reference
    from fuseml import FuseMLCompiler, FuseMLFusionPass
    from torch.fx.experimental.proxy_tensor import make_fx
    from torch.fx.passes.shape_prop import ShapeProp

    ref_file = Path(fuseml.__file__).resolve()
    assert "fuseml_b200" not in str(ref_file), "this script must import the reference, not the rebuild"

    structure = {}
    for name in configs.MAKERS:
        case = configs.make(name, small=(name != "cfg1"))
        inputs_sha = _sha(list(case.tensors.values()))
        comp = FuseMLCompiler()
        how = "reference FuseMLCompiler on CPU"
        try:
            cm = torch.compile(case.module, backend=comp)
            with torch.no_grad():
                out = cm(*case.args)
        except RuntimeError as exc:
            if "active drivers" not in str(exc):
                raise
            how = ("reference selected a Triton group (not executable without a GPU driver); "
                   "eager module output stored")
            with torch.no_grad():
                out = case.module(*case.args)
        torch._dynamo.reset()
        if not isinstance(out, (tuple, list)):
            out = (out,)
        arrays = {k: v.detach().numpy().astype(np.float32) for k, v in zip(case.outputs, out)}
        np.savez_compressed(
            HERE / f"numeric_{name}.npz",
            inputs_sha256=np.array(inputs_sha),
            how=np.array(how),
            fusion_applied=np.array(bool(comp.fusion_applied)),
            fusion_strategy=np.array(str(comp.fusion_strategy)),
            sizes=np.array(json.dumps(case.sizes)),
            **arrays,
        )
        print(name, how, comp.fusion_applied, comp.fusion_strategy, {k: v.shape for k, v in arrays.items()})

        # discovery structure on the ATen graph
        with torch.no_grad():
            gm = make_fx(lambda *a: case.module(*a))(*case.args)
        ShapeProp(gm).propagate(*case.args)
        groups = FuseMLFusionPass(gm)._find_fusion_groups()
        structure[name] = [
            {
                "op_signature": list(g.op_signature),
                "n_inputs": len(g.inputs),
                "input_shapes": [list(n.meta["tensor_meta"].shape) if "tensor_meta" in n.meta else None
                                 for n in g.inputs],
                "input_kinds": [n.op for n in g.inputs],
                "output_shape": list(g.output_metadata.get("shape", ())),
                "intermediate_outputs": len(g.intermediate_outputs),
            }
            for g in groups
        ]
        print("  groups:", [g["op_signature"] for g in structure[name]])
    (HERE / "structure.json").write_text(json.dumps(structure, indent=1) + "\n")


if __name__ == "__main__":
    main()
