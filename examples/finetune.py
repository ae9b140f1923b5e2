"""Supervised fine-tuning entry script (epoch-based loop over a json dataset of prompt / response pairs): counterpart
of the reference's finetune_utils-based launchers.

  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/finetune.py --pretrained-checkpoint /path/to/ckpt \
      --train-data-path sft.json --valid-data-path dev.json --epochs 3 --max-padding-length 2048 \
      --patch-tokenizer-type Qwen2Tokenizer --tokenizer-model /path/to/tokenizer  <model and parallelism flags>
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch                                                                       # noqa: E402

from linear_moe_b200.config.arguments import parse_args                            # noqa: E402
from linear_moe_b200.data.builders import build_datasets                           # noqa: E402
from linear_moe_b200.dist.mesh import init_distributed                             # noqa: E402
from linear_moe_b200.train.finetune import finetune                                # noqa: E402

if __name__ == "__main__":
    args, cfg, par, tc = parse_args()
    mesh = init_distributed(par)
    if tc.dataset == "Synthetic":
        tc.dataset = "LLama-SFT"                                 # json prompt/response pairs (--train-data-path / --valid-data-path)
    train_ds, valid_ds = build_datasets(args, cfg, tc)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    trainer = finetune(cfg, par, tc, train_ds, valid_ds, mesh=mesh, device=dev)
    if tc.save:
        trainer.save()
