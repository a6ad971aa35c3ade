"""A transformer patched by BlockSparseModelPatcher (reference tests/test_integration.py:66-113, README.md:54-61):
at density 1.0 the patched RoBERTa computes what the dense model computes (atol 1e-3), at density 0.5 it has
fewer parameters and trains."""
import contextlib
import io

import numpy as np
import pytest
import torch

from pytorch_block_sparse_b200 import BlockSparseLinear, BlockSparseModelPatcher

from .gpu_util import assert_device_healthy

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _roberta(layers=6):
    config = transformers.RobertaConfig(
        vocab_size=5000, max_position_embeddings=514, num_attention_heads=12, num_hidden_layers=layers,
        type_vocab_size=1, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
    )
    torch.manual_seed(0)
    return transformers.RobertaForMaskedLM(config=config).cuda()


def _patch(model, density, with_attention_output=False):
    mp = BlockSparseModelPatcher()
    mp.add_pattern("roberta\\.encoder\\.layer\\.[0-9]+.intermediate\\.dense", {"density": density})
    mp.add_pattern("roberta\\.encoder\\.layer\\.[0-9]+.output\\.dense", {"density": density})
    if with_attention_output:
        mp.add_pattern("roberta\\.encoder\\.layer\\.[0-9]+\\.attention\\.output\\.dense", {"density": density})
    with contextlib.redirect_stdout(io.StringIO()) as log:
        mp.patch_model(model)
    return log.getvalue()


def test_patched_roberta_at_full_density_equals_the_dense_model():
    np.random.seed(0)
    model = _roberta().eval()
    dense_params = model.num_parameters()
    input_ids = torch.tensor([[4, 5, 6, 7] * 8]).cuda()
    with torch.no_grad():
        out0 = model(input_ids)[0]
    log = _patch(model, 1.0)
    assert log.count("Patching with BlockSparseLinear") == 12
    sparse_layers = [m for m in model.modules() if isinstance(m, BlockSparseLinear)]
    assert len(sparse_layers) == 12
    with torch.no_grad():
        out1 = model(input_ids)[0]
    assert torch.isclose(out0, out1, atol=1e-3).all()
    assert model.num_parameters() == dense_params
    assert_device_healthy()


def test_patched_roberta_at_half_density_trains():
    np.random.seed(1)
    model = _roberta(layers=2).train()
    dense_params = model.num_parameters()
    _patch(model, 0.5, with_attention_output=True)
    assert model.num_parameters() < dense_params
    ids = torch.randint(0, 5000, (4, 64), device="cuda")
    labels = ids.clone()
    labels[:, ::2] = -100
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(8):
        opt.zero_grad(set_to_none=True)
        loss = model(input_ids=ids, labels=labels).loss
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert np.isfinite(losses).all() and losses[-1] < losses[0]
    for m in model.modules():
        if isinstance(m, BlockSparseLinear):
            assert m.weight.data.grad is not None and torch.isfinite(m.weight.data.grad).all()
    assert_device_healthy()
