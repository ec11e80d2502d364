"""Print one preset of ``configurations.yml`` as shell ``export`` lines for ``run.sub``.

    python examples/bert_pretraining/cluster_preset.py                 # list the presets
    eval "$(python examples/bert_pretraining/cluster_preset.py bert--B200_4x8x64x4)"
    sbatch -N "$NNODES" --export=ALL examples/bert_pretraining/run.sub

(The reference keeps such a file for its cluster CI, ``examples/BertPretraining/configurations.yml``.)
"""
import os
import shlex
import sys

import yaml

FILE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configurations.yml")


def load(path=FILE):
    """``{preset name: {variable: value}}``; entries whose name starts with a dot are YAML anchors only."""
    with open(path) as f:
        doc = yaml.safe_load(f)
    return {k: {n: str(v) for n, v in e["variables"].items()} for k, e in doc.items() if not k.startswith(".")}


def global_batch(v):
    return int(v["NNODES"]) * int(v["GPUS"]) * int(v["BATCH"]) * int(v["ACCUM"])


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    presets = load()
    if not argv:
        for name, v in presets.items():
            print(f"{name}: phase {v['PHASE']}, {v['NNODES']} node(s), global batch {global_batch(v)}, {v['REDUCER']}")
        return 0
    if argv[0] not in presets:
        print(f"unknown preset {argv[0]!r}; run without arguments for the list", file=sys.stderr)
        return 2
    for k, val in sorted(presets[argv[0]].items()):
        print(f"export {k}={shlex.quote(val)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
