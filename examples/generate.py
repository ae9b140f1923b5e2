"""Text generation entry: loads a checkpoint (``--load``) and completes the prompts of ``--text-generate-input-file``
(counterpart of the reference's generation scripts).  Runs in one process, or under ``torchrun`` with
``--tensor-model-parallel-size`` / ``--pipeline-model-parallel-size``: the stages relay activations, the last stage
samples and every stage receives the sampled tokens; rank 0 prints the completions.

  python examples/generate.py --load /path/to/ckpt --text-generate-input-file prompts.jsonl <model flags>
  torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/generate.py --pipeline-model-parallel-size 2 ...
  LMOE_SERVE_PORT=5000 python examples/generate.py --load /path/to/ckpt <model flags>     # serve PUT /api instead
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch                                                                      # noqa: E402

from linear_moe_b200.ckpt.legacy import load_checkpoint                           # noqa: E402
from linear_moe_b200.config.arguments import parse_args                           # noqa: E402
from linear_moe_b200.data.tokenizer import build_tokenizer                        # noqa: E402
from linear_moe_b200.dist.mesh import init_distributed, single_process_mesh       # noqa: E402
from linear_moe_b200.infer.generation import GPTPredictor                         # noqa: E402
from linear_moe_b200.models.transformer import CausalLM                           # noqa: E402

if __name__ == "__main__":
    args, cfg, par, tc = parse_args()
    distributed = int(os.environ.get("WORLD_SIZE", "1")) > 1
    if distributed:
        if not torch.cuda.is_available():
            par.distributed_backend = "gloo"
        par.sequence_parallel = False                     # one-token decode steps cannot be split along the sequence
        mesh = init_distributed(par)
    else:
        mesh = single_process_mesh()
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    tok, _ = build_tokenizer(args.patch_tokenizer_type, args.tokenizer_model, cfg.vocab_size, args.extra_vocab_size)
    model = CausalLM(cfg, mesh, pre_process=mesh.is_first_stage, post_process=mesh.is_last_stage, device=dev).to(dev)
    if tc.load:
        if tc.use_dist_ckpt:
            from linear_moe_b200.ckpt.sharded import load_sharded
            per = cfg.num_layers // mesh.pp
            load_sharded(tc.load, [model], cfg, mesh, None, layer_offsets=[mesh.pp_rank * per])
        else:
            load_checkpoint(tc.load, [model], None, None, mesh, load_rng=False)
    port = int(os.environ.get("LMOE_SERVE_PORT", "0"))
    if port:
        # HTTP endpoint (PUT /api, the request fields of Megatron's text-generation server): rank 0 serves, the other
        # ranks of a parallel replica join every generation call
        from linear_moe_b200.infer.server import build_app, serve_followers
        graph = getattr(args, "cuda_graph_decode", False)
        if mesh.rank == 0:
            import uvicorn
            uvicorn.run(build_app(model.eval(), tok, cuda_graph=graph), host=os.environ.get("LMOE_SERVE_HOST", "127.0.0.1"),
                        port=port, log_level="warning")
        else:
            serve_followers(model.eval(), tok, cuda_graph=graph)
        sys.exit(0)
    outs = GPTPredictor(model, tok, args).predict()
    if mesh.rank == 0:
        for out in outs:
            print(out)
