"""GPU: the sparse operators swapped into a LLaMA MLP block (the model-side hookup the reference
sketches in intrasm_engine/pytorch/huggingface_rewriter.py:91-170).  The block is transformers'
own ``LlamaMLP`` with random weights of a small configuration; after the swap its output and the
gradient of its input must equal those of the same block with the pruned weights kept dense."""
import copy

import pytest
import torch

from . import gpu_util as G

pytestmark = pytest.mark.gpu


def _mlp(hidden, inter, act):
    from transformers.models.llama.configuration_llama import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaMLP
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, hidden_act=act, mlp_bias=False)
    torch.manual_seed(0)
    return LlamaMLP(cfg).to(G.DEV).half()


@pytest.mark.parametrize("tokens", [64, 40])
def test_llama_mlp_with_sparse_projections(tokens):
    from intrasm_engine_b200.pytorch.huggingface_rewriter import (SparseLinear, inject_sparse_linears,
                                                                  magnitude_prune)
    dense = _mlp(256, 512, "relu")
    for p in dense.parameters():
        p.requires_grad_(False)
    sparse = copy.deepcopy(dense)
    assert inject_sparse_linears(sparse, ("up_proj", "gate_proj"), sparsity=0.6) == 2
    assert isinstance(sparse.up_proj, SparseLinear) and abs(sparse.up_proj.density() - 0.4) < 0.01
    # the dense twin keeps the same pruned weights
    for name in ("up_proj", "gate_proj"):
        getattr(dense, name).weight.copy_(magnitude_prune(getattr(dense, name).weight, 0.6))
    x1 = (torch.randn(2, tokens // 2, 256, device=G.DEV) * 0.5).half().requires_grad_(True)
    x2 = x1.detach().clone().requires_grad_(True)
    y1, y2 = sparse(x1), dense(x2)
    assert y1.shape == y2.shape == (2, tokens // 2, 256)
    assert torch.allclose(y1.float(), y2.float(), rtol=1e-2, atol=1e-2 * float(y2.abs().max()))
    g = torch.randn_like(y2)
    y1.backward(g)
    y2.backward(g)
    assert torch.allclose(x1.grad.float(), x2.grad.float(), rtol=2e-2, atol=2e-2 * float(x2.grad.abs().max()))


def test_inject_reports_missing_targets():
    from intrasm_engine_b200.pytorch.huggingface_rewriter import inject_sparse_linears
    with pytest.raises(ValueError):
        inject_sparse_linears(torch.nn.Sequential(torch.nn.Linear(8, 8)), ("q_proj",))
