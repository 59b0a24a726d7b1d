"""The fused BERT step (hand-written kernels, manual backward) against the plain PyTorch fp32 restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(tie):
    from autodist_b200.models.bert import BertConfig, BertPretrainer, synthetic_batch
    torch.manual_seed(0)
    cfg = BertConfig.tiny(tie_word_embeddings=tie, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    model = BertPretrainer(cfg)
    # larger init so that gradients are well above bf16 noise
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() == 2:
                p.normal_(0, 0.08)
    ref = BertPretrainer(cfg)
    ref.load_state_dict(model.state_dict())
    batch = synthetic_batch(cfg, batch=4, seq_len=128, max_predictions=8, seed=1)
    batch["input_mask"][:, 100:] = 0
    batch["mlm_weights"][:, -2:] = 0
    return cfg, model, ref, batch


@pytest.mark.parametrize("tie", [False, True])
def test_fused_bert_matches_reference(tie):
    cfg, model, ref, batch = _setup(tie)
    ref = ref.cuda()
    cuda_batch = {k: v.cuda() for k, v in batch.items()}
    loss_ref = ref.reference_loss(**cuda_batch)
    loss_ref.backward()
    model.materialize("cuda")
    model.training_dropout = False
    loss = model.fused_forward_backward(**cuda_batch, backward=True)
    torch.cuda.synchronize()
    model.check_error()
    assert abs(loss.item() - loss_ref.item()) < 3e-2 * abs(loss_ref.item()), (loss.item(), loss_ref.item())
    bad = []
    for (n, p), (_, pr) in zip(model.named_parameters(), ref.named_parameters()):
        g, gr = model.flat.g[n].float(), pr.grad
        denom = gr.abs().max().item() + 1e-6
        err = (g - gr).abs().max().item() / denom
        if err > 0.08:
            bad.append((n, round(err, 3), denom))
    assert not bad, bad


def test_dropout_path_runs_and_is_reproducible():
    from autodist_b200.models.bert import BertConfig, BertPretrainer, synthetic_batch
    torch.manual_seed(0)
    cfg = BertConfig.tiny()
    model = BertPretrainer(cfg)
    model.materialize("cuda")
    batch = {k: v.cuda() for k, v in synthetic_batch(cfg, 2, 128, 8).items()}
    l1 = model.fused_forward_backward(**batch).item()
    g1 = model.flat.grad.clone()
    model._ws["step"].zero_()
    l2 = model.fused_forward_backward(**batch).item()
    # same step counter -> same dropout masks; the loss and the embedding gradients are accumulated with floating-point atomics,
    # whose order may differ between two runs, so equality holds up to fp32 rounding (a different mask moves the loss by ~1e-2)
    assert abs(l1 - l2) < 1e-5 * abs(l1)
    assert (g1 - model.flat.grad).abs().max().item() <= 1e-5 * g1.abs().max().item()
    l3 = model.fused_forward_backward(**batch).item()
    assert abs(l3 - l1) > 1e-4 * abs(l1)                           # next step -> new masks
    assert torch.isfinite(model.flat.grad).all()
    model.check_error()
