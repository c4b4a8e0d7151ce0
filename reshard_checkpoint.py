"""Re-cut a saved training step for another tensor-/pipeline-parallel grid (weights, Adam moments, master weights).

    python reshard_checkpoint.py --config tmp/run/config.json --src ckpt/300 --dst ckpt_tp4/300 --tp 4 --pp 1

``--config`` is the run's config file (model shape, layer split, tying); the source grid is read off the shard file
names in ``--src``. Then set ``distributed.tp_size`` / ``pp_size`` (and, freely, ``dp_size`` / ``cp_size``) in the new run's
config and point ``checkpoint.load_path`` at ``--dst``. The reference cannot do this: its checkpoints only load on the
grid that wrote them (``picotron/checkpoint.py:232-262``).
"""
import argparse

from picotron_b200.config import load_config, resolve_model_config
from picotron_b200.reshard import grid_of, reshard_checkpoint


def _split(text):
    if text is None or text in ("reference", "balanced"):
        return text
    return [int(x) for x in text.split(",")]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True, help="config.json of the run that wrote the checkpoint")
    ap.add_argument("--src", required=True, help="directory of the saved step (holds weights_tp_rank_world_size=*.pth)")
    ap.add_argument("--dst", required=True, help="directory to write the new shards into")
    ap.add_argument("--tp", type=int, required=True, help="tensor-parallel size of the new grid")
    ap.add_argument("--pp", type=int, required=True, help="pipeline-parallel size of the new grid")
    ap.add_argument("--pp_layer_split", default=None,
                    help="layer split of the NEW grid: reference, balanced, or counts such as 17,15 (default: reference)")
    a = ap.parse_args(argv)
    cfg = load_config(a.config)
    mc = resolve_model_config(cfg)
    src_tp, src_pp = grid_of(a.src)
    paths = reshard_checkpoint(a.src, a.dst, mc, a.tp, a.pp,
                               src_layer_split=cfg["distributed"].get("pp_layer_split", "reference"),
                               dst_layer_split=_split(a.pp_layer_split) or "reference",
                               tie=bool(cfg["model"].get("tie_word_embeddings", False)))
    print(f"tp{src_tp} x pp{src_pp} -> tp{a.tp} x pp{a.pp}: wrote {len(paths)} shard(s) into {a.dst}")


if __name__ == "__main__":
    main()
