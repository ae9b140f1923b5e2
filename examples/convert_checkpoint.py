"""Checkpoint convertor: HuggingFace <-> Megatron-layout checkpoints, with TP / PP / EP splitting and merging.
Counterpart of toolkits/model_checkpoints_convertor/{qwen,llama,mistral,deepseek}/hf2mcore*.py of the reference.

  # HuggingFace directory (config.json + *.safetensors / pytorch_model*.bin) -> release checkpoint split for TP2 PP1 EP4
  python examples/convert_checkpoint.py --direction hf2mcore --load /path/to/hf --save /path/to/ckpt \
      --target-tp 2 --target-pp 1 --target-ep 4  <model flags as for pretrain.py, e.g. --base-model qwen2 --num-layers ...>
  # and back (merges whatever TP/PP/EP layout is on disk)
  python examples/convert_checkpoint.py --direction mcore2hf --load /path/to/ckpt --save /path/to/hf_out \
      --source-tp 2 --source-pp 1 --source-ep 4  <model flags>
"""
import glob
import os
import sys
from argparse import Namespace

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from linear_moe_b200.ckpt import hf_convert, legacy, reshard                      # noqa: E402
from linear_moe_b200.config.arguments import build_parser, configs_from_args       # noqa: E402


def load_hf_state_dict(path: str):
    sd = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        from safetensors.torch import load_file
        for f in files:
            sd.update(load_file(f))
        return sd
    for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
        sd.update(torch.load(f, map_location="cpu"))
    if not sd:
        raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin under {path}")
    return sd


def main():
    p = build_parser()
    p.add_argument("--direction", choices=["hf2mcore", "mcore2hf"], required=True)
    for side in ("source", "target"):
        for dim in ("tp", "pp", "ep"):
            p.add_argument(f"--{side}-{dim}", type=int, default=1)
    args = p.parse_args()
    cfg, par, tc = configs_from_args(args)
    if args.direction == "hf2mcore":
        full = hf_convert.hf_to_mcore(load_hf_state_dict(args.load), cfg)
        tp, pp, ep = args.target_tp, args.target_pp, args.target_ep
        for t in range(tp):
            for q in range(pp):
                for e in range(ep):
                    shard = reshard.shard_state_dict(full, cfg, tp, pp, ep, t, q, e)
                    path = legacy.checkpoint_name(args.save, 0, True, t, q, e, pp, ep)
                    os.makedirs(os.path.dirname(path), exist_ok=True)
                    torch.save({"args": Namespace(**vars(args)), "checkpoint_version": 3.0, "iteration": 0,
                                "model": legacy.to_reference_keys(shard)}, path)
        with open(os.path.join(args.save, "latest_checkpointed_iteration.txt"), "w") as f:
            f.write("release")
        print(f"wrote {tp * pp * ep} shard(s) under {args.save}")
    else:
        tp, pp, ep = args.source_tp, args.source_pp, args.source_ep
        it, release = legacy.read_tracker(args.load)
        shards = {}
        for t in range(tp):
            for q in range(pp):
                for e in range(ep):
                    path = legacy.checkpoint_name(args.load, it, release, t, q, e, pp, ep)
                    shards[(t, q, e)] = legacy.from_reference_keys(torch.load(path, map_location="cpu", weights_only=False)["model"])
        full = reshard.merge_state_dicts(shards, cfg, tp, pp, ep)
        hf = hf_convert.mcore_to_hf(full, cfg)
        os.makedirs(args.save, exist_ok=True)
        torch.save(hf, os.path.join(args.save, "pytorch_model.bin"))
        print(f"wrote {len(hf)} tensors to {os.path.join(args.save, 'pytorch_model.bin')}")


if __name__ == "__main__":
    main()
