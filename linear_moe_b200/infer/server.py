"""HTTP endpoint for generation: ``PUT /api`` with Megatron's text-generation-server request fields.

The reference reaches generation through ``generation/api.py::generate_and_post_process`` from batch scripts
(gpt_predictor.py:27-104); Megatron-LM pairs the same call with a small REST server (``PUT /api``:
``{"prompts": [...], "tokens_to_generate": n, "top_k": .., "top_p": .., "temperature": .., "logprobs": bool, ...}``).
This module is that endpoint on FastAPI.  Requests are served one at a time under a lock: a request is one batched
``generate_and_post_process`` call, whose decode steps replay a CUDA graph when ``cuda_graph`` is set, so there is
nothing to gain from interleaving two of them on one model replica.

    app = build_app(model, tokenizer)
    uvicorn.run(app, host="127.0.0.1", port=5000)

Under tensor / pipeline parallelism run the endpoint on rank 0 and ``serve_followers`` on the other ranks: rank 0
broadcasts every request so that all ranks enter the same collective generation call.
"""
import threading
from typing import List, Optional

import torch

from .generation import beam_search, generate_and_post_process

MAX_PROMPTS = 128
MAX_TOKENS = 4096


def _validate(req: dict) -> Optional[str]:
    """Megatron's server-side checks, as one message or None."""
    prompts = req.get("prompts")
    if not isinstance(prompts, list) or not prompts or not all(isinstance(p, str) for p in prompts):
        return "prompts must be a non-empty list of strings"
    if len(prompts) > MAX_PROMPTS:
        return f"at most {MAX_PROMPTS} prompts per request"
    n = req.get("tokens_to_generate", 64)
    if not isinstance(n, int) or n < 0 or n > MAX_TOKENS:
        return f"tokens_to_generate must be an integer in [0, {MAX_TOKENS}]"
    if n == 0 and not req.get("logprobs", False):
        return "tokens_to_generate=0 implies logprobs=True"
    k, p, t = req.get("top_k", 0), req.get("top_p", 0.0), req.get("temperature", 1.0)
    if not isinstance(k, int) or not 0 <= k <= 1000:
        return "top_k must be an integer in [0, 1000]"
    if not isinstance(p, (int, float)) or not 0.0 <= p <= 1.0:
        return "top_p must be a number in [0, 1]"
    if k > 0 and p > 0.0:
        return "cannot set both top_k and top_p"
    if not isinstance(t, (int, float)) or not 0.0 < t <= 100.0:
        return "temperature must be a positive number (at most 100)"
    b = req.get("beam_width")
    if b is not None:
        if not isinstance(b, int) or b < 1:
            return "beam_width must be a positive integer"
        if len(prompts) > 1:
            return "beam search takes one prompt per request"
    rp = req.get("repetition_penalty", 1.0)
    if not isinstance(rp, (int, float)) or rp <= 0:
        return "repetition_penalty must be positive"
    return None


def run_request(model, tokenizer, req: dict, cuda_graph: bool = False) -> dict:
    """One validated request -> response body (the collective part: every rank of a parallel model calls this)."""
    if req.get("beam_width"):
        device = next(model.parameters()).device
        ids = torch.tensor([tokenizer.tokenize(req["prompts"][0])], dtype=torch.long, device=device)
        toks, scores = beam_search(model, ids, req["beam_width"], req.get("tokens_to_generate", 64), tokenizer.eod,
                                   length_penalty=req.get("length_penalty", 1.0), num_return=req.get("beam_width"))
        return {"text": [tokenizer.decode(t) for t in toks.tolist()], "tokens": toks.tolist(), "score": scores.tolist()}
    texts, tokens, lp = generate_and_post_process(
        model, tokenizer, req["prompts"], tokens_to_generate=req.get("tokens_to_generate", 64),
        return_output_log_probs=bool(req.get("logprobs", False)), top_k_sampling=req.get("top_k", 0),
        top_p_sampling=req.get("top_p", 0.0), temperature=req.get("temperature", 1.0), add_BOS=bool(req.get("add_BOS", False)),
        use_eod_token_for_early_termination=bool(req.get("use_eod_token_for_early_termination", True)),
        repetition_penalty=req.get("repetition_penalty", 1.0), random_seed=req.get("random_seed", -1), cuda_graph=cuda_graph)
    out = {"text": texts, "tokens": tokens}
    if lp is not None:
        out["logprobs"] = [row[: max(len(t) - 1, 0)] for row, t in zip(lp.tolist(), tokens)]
    return out


def _broadcast_request(req: Optional[dict], group) -> Optional[dict]:
    import torch.distributed as dist
    box: List[Optional[dict]] = [req]
    dist.broadcast_object_list(box, src=0, group=group)
    return box[0]


def serve_followers(model, tokenizer, group=None, cuda_graph: bool = False):
    """Ranks other than 0 of a tensor- / pipeline-parallel replica: wait for rank 0's requests and join each generation
    call; a broadcast ``None`` ends the loop."""
    while True:
        req = _broadcast_request(None, group)
        if req is None:
            return
        with torch.no_grad():
            run_request(model, tokenizer, req, cuda_graph)


def build_app(model, tokenizer, cuda_graph: bool = False, group=None):
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse
    import torch.distributed as dist
    import contextlib
    lock = threading.Lock()
    parallel = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1

    @contextlib.asynccontextmanager
    async def lifespan(_app):
        yield
        if parallel:
            _broadcast_request(None, group)          # release the follower ranks

    app = FastAPI(title="linear_moe_b200 generation", lifespan=lifespan)

    @app.put("/api")
    async def api(request: Request):
        try:
            req = await request.json()
        except Exception:
            return JSONResponse({"message": "the request body must be JSON"}, status_code=400)
        if not isinstance(req, dict):
            return JSONResponse({"message": "the request body must be a JSON object"}, status_code=400)
        err = _validate(req)
        if err is not None:
            return JSONResponse({"message": err}, status_code=400)
        with lock, torch.no_grad():
            if parallel:
                _broadcast_request(req, group)
            return run_request(model, tokenizer, req, cuda_graph)

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    return app
