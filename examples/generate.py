"""Text generation / evaluation entry: loads a checkpoint (``--load``) and completes the prompts of
``--text-generate-input-file`` (counterpart of the reference's evaluate_*/generation scripts)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from linear_moe_b200.ckpt.legacy import load_checkpoint
from linear_moe_b200.config.arguments import parse_args
from linear_moe_b200.data.tokenizer import build_tokenizer
from linear_moe_b200.dist.mesh import single_process_mesh
from linear_moe_b200.infer.generation import GPTPredictor
from linear_moe_b200.models.transformer import CausalLM

if __name__ == "__main__":
    args, cfg, par, tc = parse_args()
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    tok, _ = build_tokenizer(args.patch_tokenizer_type, args.tokenizer_model, cfg.vocab_size, args.extra_vocab_size)
    model = CausalLM(cfg, single_process_mesh(), device=dev).to(dev)
    if tc.load:
        load_checkpoint(tc.load, [model], None, None, single_process_mesh(), load_rng=False)
    for out in GPTPredictor(model, tok, args).predict():
        print(out)
