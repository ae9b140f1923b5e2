"""Activation offload: gradients equal the plain run; one copy per distinct tensor; buffers recycled; micro-batches kept apart."""
import pytest
import torch

from linear_moe_b200.parallel.offload import ActivationOffload


class _Blocks(torch.nn.Module):
    def __init__(self, n, h):
        super().__init__()
        self.layers = torch.nn.ModuleList([torch.nn.Sequential(torch.nn.Linear(h, 2 * h), torch.nn.GELU(), torch.nn.Linear(2 * h, h))
                                           for _ in range(n)])

    def forward(self, x, off=None):
        for i, l in enumerate(self.layers):
            if off is None:
                x = x + l(x)
            else:
                with off.layer(i):
                    x = x + l(x)
        return x


def _grads(m):
    return [p.grad.clone() for p in m.parameters()]


def _run(device, dtype=torch.float32):
    torch.manual_seed(0)
    m = _Blocks(4, 64).to(device=device, dtype=dtype)
    x = torch.randn(8, 128, 64, device=device, dtype=dtype, requires_grad=True)
    m(x).square().mean().backward()
    ref, xg = _grads(m), x.grad.clone()
    m.zero_grad()
    x.grad = None
    off = ActivationOffload(3, min_bytes=1024, offload_cpu_tensors=(device == "cpu"))
    for step in range(2):                                   # the second step reuses the pooled host buffers
        m.zero_grad()
        x.grad = None
        m(x, off).square().mean().backward()
        for a, b in zip(_grads(m), ref):
            torch.testing.assert_close(a, b, rtol=0, atol=0)
        torch.testing.assert_close(x.grad, xg, rtol=0, atol=0)
        assert not off._groups, "every group is recycled once its backward ran"
        if step == 0:
            pooled = off.pinned_bytes()
            assert pooled > 0
    assert off.pinned_bytes() == pooled, "no new host buffers after the first step"
    assert off.stats["packed"] > 0 and off.stats["prefetched"] > 0
    return off


def test_offload_matches_plain_cpu():
    off = _run("cpu")
    assert off.stats["kept"] > 0                            # parameters and weight views stay where they are


def test_offload_dedupes_same_tensor():
    off = ActivationOffload(1, min_bytes=0, offload_cpu_tensors=True)
    x = torch.randn(64, 64, requires_grad=True)
    with off.layer(0):
        h = x * 2.0
        y = h.sin() + h.cos()                               # both save h
    y.sum().backward()
    assert off.stats["deduped"] >= 1
    torch.testing.assert_close(x.grad, 2.0 * ((x * 2).cos() - (x * 2).sin()))


def test_offload_microbatches_interleaved():
    """Two forwards before the backwards (1F1B): groups of the two micro-batches do not mix."""
    torch.manual_seed(1)
    m = _Blocks(2, 32)
    xs = [torch.randn(4, 16, 32, requires_grad=True) for _ in range(2)]
    ref = []
    for x in xs:
        m.zero_grad()
        m(x).square().mean().backward()
        ref.append((_grads(m), x.grad.clone()))
        x.grad = None
    off = ActivationOffload(2, min_bytes=0, offload_cpu_tensors=True)
    outs = [m(x, off).square().mean() for x in xs]
    for i in (0, 1):
        m.zero_grad()
        outs[i].backward()
        for a, b in zip(_grads(m), ref[i][0]):
            torch.testing.assert_close(a, b, rtol=0, atol=0)
        torch.testing.assert_close(xs[i].grad, ref[i][1], rtol=0, atol=0)
    off.step_done()
    assert not off._groups


@pytest.mark.gpu
def test_offload_matches_plain_gpu():
    off = _run("cuda", torch.bfloat16)
    assert off.stats["bytes"] > 0


@pytest.mark.gpu
def test_offload_model_gpu():
    """A small LSM model trains to the same loss with and without offload of its first block."""
    from linear_moe_b200.config.model_config import ModelConfig
    from linear_moe_b200.models.transformer import CausalLM
    losses = []
    for offl in (False, True):
        torch.manual_seed(0)
        cfg = ModelConfig(num_layers=2, hidden_size=256, num_attention_heads=2, ffn_hidden_size=512, vocab_size=512,
                          use_la_module=True, la_module="gla", layer_type_list="LL", params_dtype=torch.bfloat16,
                          cpu_offloading=offl,
                          cpu_offloading_num_layers=1)
        m = CausalLM(cfg, device="cuda").cuda().train()
        ids = torch.randint(0, 512, (2, 2048), device="cuda")
        loss = m(ids, labels=ids).float().mean()
        loss.backward()
        losses.append((loss.item(), m.decoder.layers[0].mlp.linear_fc2.weight.grad.float().norm().item()
                       if m.decoder.layers[0].mlp.linear_fc2.weight.grad is not None else 0.0))
        if offl:
            assert m.offload.stats["packed"] > 0
    assert abs(losses[0][0] - losses[1][0]) < 1e-6 and abs(losses[0][1] - losses[1][1]) <= 1e-3 * max(losses[0][1], 1e-6)


def test_offload_flags_reach_the_model():
    """``--cpu-offloading --cpu-offloading-num-layers N`` (the reference's TransformerEngine offload flags) build a model
    whose first N blocks run under the offload context; training-mode forward + backward on CPU leaves gradients equal
    to the plain model's."""
    from linear_moe_b200.config.arguments import build_parser, configs_from_args
    from linear_moe_b200.models.transformer import CausalLM
    base = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "2", "--ffn-hidden-size", "128",
            "--seq-length", "64", "--max-position-embeddings", "64", "--micro-batch-size", "1", "--global-batch-size", "1",
            "--use-la-module", "--la-module", "gla", "--layer-type-list", "LL", "--vocab-size", "128"]
    grads = []
    for extra in ([], ["--cpu-offloading", "--cpu-offloading-num-layers", "1"]):
        args = build_parser().parse_args(base + extra)
        cfg, _, _ = configs_from_args(args)
        assert cfg.cpu_offloading == bool(extra)
        torch.manual_seed(0)
        m = CausalLM(cfg).float().train()
        if extra:
            assert m.offload is not None and m.offload.num_layers == 1
            m.offload.min_bytes, m.offload.offload_cpu_tensors = 0, True
        ids = torch.randint(0, 128, (1, 64), generator=torch.Generator().manual_seed(1))
        m(ids, labels=ids).float().mean().backward()
        if extra:
            assert m.offload.stats["packed"] > 0
        grads.append([p.grad.clone() for p in m.parameters() if p.grad is not None])
    assert len(grads[0]) == len(grads[1])
    for a, b in zip(*grads):
        torch.testing.assert_close(a, b, rtol=0, atol=0)
