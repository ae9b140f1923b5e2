"""CPU oracle tests of the remaining reference operators: softmax attention (GQA, query offset, sliding window), norms,
RoPE, causal convolution with its decoding state, cross-entropy, feature maps and the hybrid layer allocator."""
import math

import pytest
import torch
import torch.nn.functional as F

from linear_moe_b200.models import feature_maps as FM
from linear_moe_b200.models import layout
from linear_moe_b200.ref import ops as R


def test_softmax_attention_matches_sdpa_and_offsets():
    torch.manual_seed(0)
    B, T, Hq, Hkv, D = 2, 33, 4, 2, 16
    q, k, v = torch.randn(B, T, Hq, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
    o = R.softmax_attention(q, k, v)
    ref = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(2, 1),
                                         v.transpose(1, 2).repeat_interleave(2, 1), is_causal=True).transpose(1, 2)
    assert torch.allclose(o, ref, atol=1e-5)
    # a suffix of the queries with q_offset equals the same rows of the full result (sequence-parallel / decoding form)
    o_tail = R.softmax_attention(q[:, 20:], k, v, q_offset=20)
    assert torch.allclose(o_tail, o[:, 20:], atol=1e-5)
    # a sliding window of the whole length is plain causal attention; window 1 returns v of the same position
    assert torch.allclose(R.softmax_attention(q, k, v, window=T), o, atol=1e-6)
    o1 = R.softmax_attention(q, k, v, window=1)
    assert torch.allclose(o1, v.repeat_interleave(2, 2), atol=1e-6)


def test_norms():
    torch.manual_seed(1)
    x, w = torch.randn(5, 7, 32), torch.rand(32) + 0.5
    y = R.rms_norm(x, w, eps=1e-6)
    assert torch.allclose(y, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w, atol=1e-6)
    z = torch.randn(5, 7, 32)
    g = R.gated_rms_norm(x, z, w, eps=1e-5)
    assert torch.allclose(g, R.rms_norm(x * F.silu(z), w, eps=1e-5), atol=1e-5)
    n = R.l2_norm(x)
    assert torch.allclose(n.norm(dim=-1), torch.ones(5, 7), atol=1e-4)
    s = R.swiglu(torch.cat([x, z], -1))
    assert torch.allclose(s, F.silu(x) * z, atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    torch.manual_seed(2)
    B, T, H, D = 1, 20, 2, 16
    q, k = torch.randn(B, T, H, D), torch.randn(B, T, H, D)
    cos, sin = R.rope_freqs(T, D)
    for inter in (False, True):
        qr, kr = R.apply_rope(q, cos, sin, inter), R.apply_rope(k, cos, sin, inter)
        assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-5)            # a rotation keeps the norm
        # scores depend on the distance only: shifting both positions by 5 leaves q_i . k_j unchanged
        cos5, sin5 = R.rope_freqs(T, D, offset=5)
        q5, k5 = R.apply_rope(q, cos5, sin5, inter), R.apply_rope(k, cos5, sin5, inter)
        s0 = torch.einsum("bihd,bjhd->bhij", qr, kr)
        s5 = torch.einsum("bihd,bjhd->bhij", q5, k5)
        assert torch.allclose(s0, s5, atol=1e-4)
    # partial rotary: channels beyond the table's width pass through
    cos8, sin8 = R.rope_freqs(T, 8)
    assert torch.equal(R.apply_rope(q, cos8, sin8)[..., 8:], q[..., 8:])
    # YaRN with factor 1 is plain RoPE with unit magnitude scale
    c, s, m = R.yarn_freqs(T, D, 10000.0, 1.0)
    assert torch.allclose(c, cos, atol=1e-6) and torch.allclose(s, sin, atol=1e-6) and m == 1.0


def test_causal_conv_state_chaining():
    torch.manual_seed(3)
    B, T, D, K = 2, 19, 6, 4
    x, w, b = torch.randn(B, T, D), torch.randn(D, K), torch.randn(D)
    y, st = R.causal_conv1d(x, w, b)
    ref = F.silu(F.conv1d(F.pad(x.transpose(1, 2), (K - 1, 0)), w[:, None, :], b, groups=D).transpose(1, 2))
    assert torch.allclose(y, ref, atol=1e-5)
    assert torch.equal(st, x[:, T - (K - 1):])
    y1, s1 = R.causal_conv1d(x[:, :11], w, b)
    y2, s2 = R.causal_conv1d(x[:, 11:], w, b, initial_state=s1)
    assert torch.allclose(torch.cat([y1, y2], 1), y, atol=1e-6) and torch.equal(s2, st)


def test_linear_cross_entropy_ignores_labels():
    torch.manual_seed(4)
    h, w = torch.randn(10, 8), torch.randn(12, 8)
    labels = torch.randint(0, 12, (10,))
    labels[3] = -100
    loss = R.linear_cross_entropy(h, w, labels)
    assert loss[3] == 0
    lp = torch.log_softmax(h @ w.t(), -1)
    keep = labels != -100
    assert torch.allclose(loss[keep], -lp[keep].gather(1, labels[keep][:, None])[:, 0], atol=1e-5)


def test_taylor_feature_map_approximates_exp():
    """phi(q).phi(k) = 1 + s + s^2/2 with s = q.k/sqrt(d): the second-order Taylor series of exp(s) (Based)."""
    torch.manual_seed(5)
    d = 8
    q, k = torch.randn(50, d) * 0.5, torch.randn(50, d) * 0.5
    fm = FM.build_feature_map("taylor", d)
    s = (q * k).sum(-1) / math.sqrt(d)
    assert torch.allclose((fm(q) * fm(k)).sum(-1), 1 + s + s * s / 2, atol=1e-5)


def test_rebased_feature_map_is_a_squared_kernel():
    """phi(q).phi(k) = (q'.k')^2 / d for the layer-normed q', k' (Rebased)."""
    torch.manual_seed(6)
    d = 8
    fm = FM.build_feature_map("rebased", d)
    q, k = torch.randn(30, d), torch.randn(30, d)
    qn, kn = fm(q, flatten=False), fm(k, flatten=False)
    assert torch.allclose((fm(q) * fm(k)).sum(-1), (qn * kn).sum(-1).pow(2) / d, atol=1e-4)


@pytest.mark.parametrize("name", ["elu", "relu", "identity", "swish", "sigmoid", "gelu", "sqrelu", "hedgehog", "t2r",
                                  "elementwise_product", "dpfp", "taylor", "rebased"])
def test_feature_maps_build_and_backprop(name):
    torch.manual_seed(7)
    fm = FM.build_feature_map(name, 16)
    x = torch.randn(2, 5, 3, 16, requires_grad=True)
    y = fm(x)
    assert y.shape[:-1] == x.shape[:-1] and torch.isfinite(y).all()
    y.sum().backward()
    assert torch.isfinite(x.grad).all()


def test_hybrid_layer_allocator():
    """Attention and MLP blocks are spread evenly among the Mamba blocks and counts follow the ratios."""
    p = layout.allocate_mamba_pattern(16, 0.25, 0.0)
    assert p.count("*") == 4 and p.count("M") == 12
    gaps = [i for i, s in enumerate(p) if s == "*"]
    assert max(b - a for a, b in zip(gaps, gaps[1:])) - min(b - a for a, b in zip(gaps, gaps[1:])) <= 1
    p = layout.allocate_mamba_pattern(24, 0.125, 0.25)
    assert (p.count("*"), p.count("-"), p.count("M")) == (3, 6, 15)
    assert layout.allocate_mamba_pattern(4, 0.0, 0.0, override="M*-M") == list("M*-M")
    with pytest.raises(ValueError):
        layout.allocate_mamba_pattern(4, 0.0, 0.0, override="M*-")
    with pytest.raises(ValueError):
        layout.allocate_mamba_pattern(4, 0.0, 0.0, override="MxMM")
    with pytest.raises(ValueError):
        layout.allocate_mamba_pattern(4, 0.5, 0.0, override="MMMM")


def test_rope_with_sequence_offsets_and_packed_sequences():
    """Rotary embedding with per-sequence start offsets and with packed sequences (positions restart at cu_seqlens
    boundaries) equals the plain op applied to each sequence with its own table slice."""
    import torch
    from linear_moe_b200 import ops
    from linear_moe_b200.ref import ops as R
    torch.manual_seed(0)
    B, T, H, D = 3, 10, 2, 16
    cos, sin = R.rope_freqs(64, D, 10000.0, 0, torch.device("cpu"), None)
    x = torch.randn(B, T, H, D)
    offs = torch.tensor([0, 5, 17])
    pos = ops.rope_positions(T, B, x.device, seqlen_offsets=offs)
    got = ops.apply_rope_at(x, cos, sin, pos)
    for b in range(B):
        o = int(offs[b])
        want = ops.apply_rope(x[b:b + 1], cos[o:o + T], sin[o:o + T])
        assert torch.allclose(got[b:b + 1], want, atol=1e-6)
    assert torch.equal(ops.rope_positions(T, B, x.device, seqlen_offsets=4), torch.arange(4, 4 + T).expand(B, T))
    # packed: three sequences of 4, 1 and 7 tokens in one row of 12
    cu = torch.tensor([0, 4, 5, 12])
    xp = torch.randn(1, 12, H, D)
    pos = ops.rope_positions(12, 1, xp.device, cu_seqlens=cu)
    assert pos.tolist() == [[0, 1, 2, 3, 0, 0, 1, 2, 3, 4, 5, 6]]
    got = ops.apply_rope_at(xp, cos, sin, pos, interleaved=True)
    for s, e in zip(cu[:-1].tolist(), cu[1:].tolist()):
        want = ops.apply_rope(xp[:, s:e], cos[: e - s], sin[: e - s], interleaved=True)
        assert torch.allclose(got[:, s:e], want, atol=1e-6)
    pos = ops.rope_positions(12, 1, xp.device, cu_seqlens=cu, seqlen_offsets=torch.tensor([2, 0, 9]))
    assert pos.tolist() == [[2, 3, 4, 5, 0, 9, 10, 11, 12, 13, 14, 15]]


def test_vocab_parallel_ce_label_mapping():
    """Label tensors handed to the per-shard softmax kernels of the vocabulary-parallel cross entropy: the local column
    inside the shard, the ignore value for ignored rows, and a value that matches no column for targets in other shards."""
    import torch
    from linear_moe_b200.parallel.tensor_parallel import _ce_kernel_labels
    labels = torch.tensor([0, 5, 9, 10, 19, 20, -100, 15])
    inshard, fwd, bwd = _ce_kernel_labels(labels, vocab_start=10, width=10, ignore_index=-100)
    assert inshard.tolist() == [False, False, False, True, True, False, False, True]
    assert fwd.tolist() == [-100, -100, -100, 0, 9, -100, -100, 5]           # the forward kernel reads logit[label]: in-shard only
    assert bwd.tolist() == [-1, -1, -1, 0, 9, -1, -100, 5]                   # -1: softmax part only; -100: no gradient
    _, _, bwd2 = _ce_kernel_labels(torch.tensor([3, -1]), 0, 2, ignore_index=-1)
    assert bwd2.tolist() == [-2, -1]                                          # the "nowhere" value never equals the ignore value
