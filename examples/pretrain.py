"""Training entry script: the counterpart of examples/*/pretrain_{qwen,llama,mistral,deepseek}.py of the reference.
All four backbones and every ``--la-module`` go through this one script; the backbone is ``--base-model``.

  torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/pretrain.py --base-model qwen2 --use-la-module \
      --la-module gla --layer-type-list LLLNLLLNLLLN ...
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from linear_moe_b200.train.loop import pretrain

if __name__ == "__main__":
    pretrain()
