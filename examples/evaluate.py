"""Evaluation entry script: validation loss / perplexity of a checkpoint, and an lm-evaluation-harness run when the
`lm_eval` package is installed.  Counterpart of examples/linear_moe_qwen2/evaluate_mcore_qwen.py and
eval/lm_eval_linear_moe.sh of the reference.

  torchrun --nproc-per-node 1 --master-addr 127.0.0.1 examples/evaluate.py --load /path/to/ckpt --eval-iters 50 \
      --dataset LLama-Pretrain-Idxmap --data-path corpus_text_document  <model flags>
  python examples/evaluate.py --load /path/to/ckpt --lm-eval-tasks piqa,hellaswag \
      --patch-tokenizer-type Qwen2Tokenizer --tokenizer-model /path/to/tokenizer  <model flags>
"""
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch                                                                       # noqa: E402

from linear_moe_b200.config.arguments import build_parser, configs_from_args       # noqa: E402
from linear_moe_b200.data.builders import build_datasets                           # noqa: E402
from linear_moe_b200.dist.mesh import init_distributed                             # noqa: E402
from linear_moe_b200.train.loop import Trainer                                     # noqa: E402

if __name__ == "__main__":
    p = build_parser()
    p.add_argument("--lm-eval-tasks", type=str, default=None, help="comma-separated lm-evaluation-harness task names")
    args = p.parse_args()
    import logging
    logging.basicConfig(level=getattr(logging, str(args.verbosity).upper(), logging.INFO))      # --verbosity (lm_evaluate.py)
    cfg, par, tc = configs_from_args(args)
    mesh = init_distributed(par)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    tc.no_load_optim, tc.no_load_rng = True, True
    train_ds, valid_ds = build_datasets(args, cfg, tc)
    trainer = Trainer(cfg, par, tc, mesh, device=dev, dataset=train_ds, valid_dataset=valid_ds or train_ds)
    if args.lm_eval_tasks:
        try:
            import lm_eval
        except ImportError:
            raise SystemExit("lm_eval is not installed; install lm-evaluation-harness to run --lm-eval-tasks")
        from linear_moe_b200.data.tokenizer import build_tokenizer
        from linear_moe_b200.infer.lm_eval_adaptor import get_lm_eval_model
        tok, _ = build_tokenizer(args.patch_tokenizer_type, args.tokenizer_model, cfg.vocab_size, args.extra_vocab_size)
        lm = get_lm_eval_model(trainer.model, tok)
        tasks = args.lm_eval_tasks.split(",") if args.lm_eval_tasks != "all" else args.task_list.split(",")
        res = lm_eval.simple_evaluate(model=lm, tasks=tasks, num_fewshot=args.num_fewshot)
        if mesh.rank == 0:
            print(res["results"])
    else:
        stats = trainer.evaluate(tc.eval_iters)
        if mesh.rank == 0 and stats:
            loss = float(stats.get("lm loss", float("nan")))
            print(f"validation loss {loss:.6f} | perplexity {math.exp(min(loss, 20.0)):.4f}")
