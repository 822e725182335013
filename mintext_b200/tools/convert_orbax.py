"""Convert between the reference's Orbax checkpoints and this framework's checkpoint layout.

    python -m mintext_b200.tools.convert_orbax from-orbax <orbax_dir>/<step>/default  <out_checkpoint_dir> [--step N]
    python -m mintext_b200.tools.convert_orbax to-orbax   <checkpoint_dir> <step>      <orbax_out_dir>

The reference saves its whole ``TrainState`` (``step``, ``params``, ``opt_state``) with Orbax ``StandardSave``
(mintext/checkpoint/manager.py:54-74), i.e. as an OCDBT / TensorStore tree.  Reading or writing that format needs the
``orbax-checkpoint`` package (and its TensorStore dependency), which this build's machines do not have; the tool is
meant to be run wherever Orbax is installed - typically next to the reference - and imports it only then.  Everything
apart from the two Orbax calls (tree flattening, the path mapping between the two trees, reading and writing this
framework's own layout) is plain Python + numpy and is tested without Orbax.

Tree mapping.  The reference's parameter tree is the Flax NNX state: nested dicts keyed by attribute names and layer
indices, each leaf wrapped as ``{"value": array}``.  Here a parameter is ``params/<dotted module path>``.  So
``params/layers/3/attention/query/kernel/value`` <-> ``params/layers.3.attention.query.kernel``.  Optimizer moments are
found by name: any subtree of ``opt_state`` called ``mu`` / ``nu`` whose inner paths mirror the parameter tree maps to
``opt_state/mu/<name>`` / ``opt_state/nu/<name>``; the step counter to ``step`` and ``opt_state/count``.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np


# ------------------------------------------------------------------------------------------ pure tree handling
def flatten_tree(tree, prefix: tuple = ()) -> dict[tuple, np.ndarray]:
    """Nested dicts / lists -> ``{path tuple: leaf}`` (list positions become their index as a string)."""
    out: dict[tuple, np.ndarray] = {}
    if isinstance(tree, dict):
        for k, v in tree.items():
            out.update(flatten_tree(v, prefix + (str(k),)))
    elif isinstance(tree, (list, tuple)):
        for i, v in enumerate(tree):
            out.update(flatten_tree(v, prefix + (str(i),)))
    elif tree is not None:
        out[prefix] = tree
    return out


def unflatten_tree(flat: dict[tuple, object]) -> dict:
    root: dict = {}
    for path, leaf in flat.items():
        node = root
        for p in path[:-1]:
            node = node.setdefault(p, {})
        node[path[-1]] = leaf
    return root


def _strip_value(path: tuple) -> tuple:
    return path[:-1] if path and path[-1] in ("value", "raw_value") else path


def orbax_to_native(tree: dict) -> dict[str, np.ndarray]:
    """Flat ``{native path: array}`` from a restored reference ``TrainState`` tree."""
    out: dict[str, np.ndarray] = {}
    flat = {_strip_value(p): v for p, v in flatten_tree(tree).items()}
    for path, leaf in flat.items():
        arr = np.asarray(leaf)
        if path and path[0] == "params":
            out["params/" + ".".join(path[1:])] = arr
        elif path == ("step",):
            out["step"] = arr
        elif path and path[0] == "opt_state":
            for kind in ("mu", "nu"):
                if kind in path[1:]:
                    i = path.index(kind, 1)
                    out[f"opt_state/{kind}/" + ".".join(path[i + 1:])] = arr
                    break
            else:
                if path[-1] == "count" and "opt_state/count" not in out:
                    out["opt_state/count"] = arr
    if "step" in out and "opt_state/count" not in out:
        out["opt_state/count"] = out["step"]
    return out


def native_to_orbax(flat: dict[str, np.ndarray]) -> dict:
    """Nested reference-style tree from native paths (moments go under ``opt_state/{mu,nu}``, leaves as ``value``)."""
    tree: dict[tuple, object] = {}
    for path, arr in flat.items():
        head, _, name = path.partition("/")
        if head == "params":
            tree[("params",) + tuple(name.split(".")) + ("value",)] = arr
        elif head == "opt_state":
            kind, _, rest = name.partition("/")
            if kind in ("mu", "nu"):
                tree[("opt_state", kind) + tuple(rest.split(".")) + ("value",)] = arr
            else:
                tree[("opt_state", kind)] = arr
        else:
            tree[(head,)] = arr
    return unflatten_tree(tree)


# ------------------------------------------------------------------------------------------ this framework's layout
class _DictState:
    """Adapter that lets the checkpoint manager write / read a flat ``{path: array}`` dict."""

    def __init__(self, flat: dict | None = None):
        self.flat = dict(flat or {})

    def checkpoint_tree(self) -> dict:
        import torch

        out = {}
        for k, v in self.flat.items():
            a = np.asarray(v)
            out[k] = int(a) if (a.ndim == 0 and a.dtype.kind in "iu") else torch.from_numpy(np.ascontiguousarray(a))
        return out

    def load_checkpoint_tree(self, read) -> None:
        import torch

        for k in read.paths:
            v = read(k)
            if isinstance(v, torch.Tensor):
                v = v.float().numpy() if v.dtype == torch.bfloat16 else v.numpy()
            if not isinstance(v, str):  # layout descriptions of the flat-buffer engine are not part of the exchange
                self.flat[k] = np.asarray(v)


def write_native(flat: dict[str, np.ndarray], directory: str, step: int) -> None:
    from mintext_b200.checkpoint.manager import CheckpointManager

    m = CheckpointManager(directory, enable_async=False)
    m.save(step, _DictState(flat), force=True)
    m.wait_until_finished()


def read_native(directory: str, step: int) -> dict[str, np.ndarray]:
    from mintext_b200.checkpoint.manager import CheckpointManager

    st = _DictState()
    CheckpointManager(directory, read_only=True).restore(step, st)
    return st.flat


# ------------------------------------------------------------------------------------------ the two Orbax calls
def _orbax():
    try:
        import orbax.checkpoint as ocp
    except ImportError as e:  # pragma: no cover - depends on the machine
        raise SystemExit("this conversion needs the `orbax-checkpoint` package; run it where the reference's "
                         f"environment is installed ({e})")
    return ocp


def load_orbax_tree(path: str) -> dict:  # pragma: no cover - needs orbax
    ocp = _orbax()
    return ocp.PyTreeCheckpointer().restore(str(Path(path).resolve()))


def save_orbax_tree(tree: dict, path: str) -> None:  # pragma: no cover - needs orbax
    ocp = _orbax()
    ocp.PyTreeCheckpointer().save(str(Path(path).resolve()), tree)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("from-orbax", help="reference Orbax step directory -> this framework's checkpoint directory")
    a.add_argument("orbax_path")
    a.add_argument("out_dir")
    a.add_argument("--step", type=int, default=None, help="step number to write (default: the tree's `step`)")
    b = sub.add_parser("to-orbax", help="a step of this framework's checkpoint directory -> an Orbax tree")
    b.add_argument("checkpoint_dir")
    b.add_argument("step", type=int)
    b.add_argument("orbax_out")
    args = ap.parse_args(argv)
    if args.cmd == "from-orbax":
        flat = orbax_to_native(load_orbax_tree(args.orbax_path))
        step = args.step if args.step is not None else int(np.asarray(flat.get("step", 0)))
        write_native(flat, args.out_dir, step)
        print(json.dumps({"written": args.out_dir, "step": step, "entries": len(flat)}))
    else:
        flat = read_native(args.checkpoint_dir, args.step)
        save_orbax_tree(native_to_orbax(flat), args.orbax_out)
        print(json.dumps({"written": args.orbax_out, "entries": len(flat)}))


if __name__ == "__main__":
    main()
