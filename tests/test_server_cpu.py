"""The generation endpoint (infer/server.py) through FastAPI's test client."""
import pytest
import torch

from linear_moe_b200.config.model_config import ModelConfig
from linear_moe_b200.data.tokenizer import NullTokenizer
from linear_moe_b200.infer import generation as G
from linear_moe_b200.infer.server import build_app
from linear_moe_b200.models.transformer import CausalLM


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from linear_moe_b200.parallel.tensor_parallel import set_init_seed
    set_init_seed(1234)             # earlier tests in the same process may have trained with another seed
    torch.manual_seed(0)
    cfg = ModelConfig(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, vocab_size=128,
                      use_la_module=True, la_module="gla", layer_type_list="LN", init_method_std=0.1)
    model = CausalLM(cfg).eval()
    tok = NullTokenizer(128)
    with TestClient(build_app(model, tok)) as c:
        yield c, model, tok


def test_greedy_request_matches_the_library_call(client):
    c, model, tok = client
    body = {"prompts": ["1 2 3 4", "9 8 7 6 5 4"], "tokens_to_generate": 5, "top_k": 1, "logprobs": True}
    r = c.put("/api", json=body)
    assert r.status_code == 200, r.text
    out = r.json()
    with torch.no_grad():
        texts, tokens, lp = G.generate_and_post_process(model, tok, body["prompts"], 5, top_k_sampling=1,
                                                        return_output_log_probs=True)
    assert out["text"] == texts and out["tokens"] == tokens
    assert len(out["logprobs"]) == 2 and len(out["logprobs"][0]) == len(tokens[0]) - 1
    assert abs(out["logprobs"][1][2] - float(lp[1, 2])) < 1e-5
    assert c.get("/health").json() == {"status": "ok"}


def test_scoring_and_beam_requests(client):
    c, model, tok = client
    r = c.put("/api", json={"prompts": ["5 6 7 8 9"], "tokens_to_generate": 0, "logprobs": True})
    assert r.status_code == 200 and len(r.json()["logprobs"][0]) == 4
    r = c.put("/api", json={"prompts": ["5 6 7"], "tokens_to_generate": 4, "beam_width": 3})
    out = r.json()
    assert r.status_code == 200 and len(out["text"]) == 3 and out["score"] == sorted(out["score"], reverse=True)
    assert all(t[:3] == [5, 6, 7] for t in out["tokens"])


@pytest.mark.parametrize("body,needle", [
    ({"prompts": []}, "non-empty"), ({"prompts": "1 2"}, "list of strings"),
    ({"prompts": ["1"], "tokens_to_generate": -1}, "tokens_to_generate"),
    ({"prompts": ["1"], "tokens_to_generate": 0}, "implies logprobs"),
    ({"prompts": ["1"], "top_k": 2, "top_p": 0.5}, "both top_k and top_p"),
    ({"prompts": ["1"], "temperature": 0}, "temperature"),
    ({"prompts": ["1", "2"], "beam_width": 2}, "one prompt"),
    ({"prompts": ["1"], "top_p": 1.5}, "top_p"),
])
def test_bad_requests_are_refused_with_a_message(client, body, needle):
    c, _, _ = client
    r = c.put("/api", json=body)
    assert r.status_code == 400 and needle in r.json()["message"]
    assert c.put("/api", content=b"not json").status_code == 400


def _parallel_worker(rank, world):
    from linear_moe_b200.config.model_config import ParallelConfig
    from linear_moe_b200.dist.mesh import Mesh
    from linear_moe_b200.infer import server as S
    from linear_moe_b200.parallel.tensor_parallel import set_init_seed
    set_init_seed(1234)
    mesh = Mesh(ParallelConfig(distributed_backend="gloo", tensor_model_parallel_size=2))
    cfg = ModelConfig(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, vocab_size=128,
                      use_la_module=True, la_module="gla", layer_type_list="LN", init_method_std=0.1)
    model, tok = CausalLM(cfg, mesh).eval(), NullTokenizer(128)
    if rank != 0:
        S.serve_followers(model, tok)
        return None
    outs = []
    with torch.no_grad():
        for req in ({"prompts": ["1 2 3 4"], "tokens_to_generate": 4, "top_k": 1},
                    {"prompts": ["7 7 7", "3 2 1 0 9"], "tokens_to_generate": 3, "top_k": 1, "logprobs": True}):
            S._broadcast_request(req, None)
            outs.append(S.run_request(model, tok, req))
    S._broadcast_request(None, None)
    return outs


def test_follower_ranks_join_every_request(client):
    """A tensor-parallel replica: rank 0 hands each request to the follower loop of rank 1 and both generate together;
    the tokens equal those of the single-process model."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed
    c, _, _ = client
    outs = run_distributed(_parallel_worker, 2)[0]
    one = c.put("/api", json={"prompts": ["1 2 3 4"], "tokens_to_generate": 4, "top_k": 1}).json()
    two = c.put("/api", json={"prompts": ["7 7 7", "3 2 1 0 9"], "tokens_to_generate": 3, "top_k": 1, "logprobs": True}).json()
    assert outs[0]["tokens"] == one["tokens"] and outs[1]["tokens"] == two["tokens"]
    assert abs(outs[1]["logprobs"][1][3] - two["logprobs"][1][3]) < 1e-4
