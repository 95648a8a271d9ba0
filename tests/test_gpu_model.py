"""End-to-end native training path on the GPU against the eager fp32 model."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(vocab_size=1003, context_length=256, d_model=256, num_layers=2, num_heads=4, d_ff=688, rope_theta=10000.0)


def _models():
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    torch.manual_seed(0)
    eager = TransformerLM(**CFG).cuda()
    native = TransformerLM(**CFG, use_custom_triton=True).cuda()
    native.load_state_dict(eager.state_dict())
    return eager, native


def test_logits_loss_and_grads_close_to_fp32():
    from llm_systems_from_scratch_b200.ops import native as nat
    eager, native = _models()
    x = torch.randint(0, CFG["vocab_size"], (3, 200), device="cuda")
    y = torch.randint(0, CFG["vocab_size"], (3, 200), device="cuda")
    le = eager(x)
    ln = native(x)
    nat.check_status()
    assert ln.shape == le.shape and ln.dtype == torch.bfloat16
    assert (ln.float() - le).abs().max().item() < 0.15
    ref = torch.nn.functional.cross_entropy(le.view(-1, le.shape[-1]), y.view(-1))
    ref.backward()
    loss = native.loss(x, y)
    loss.backward()
    nat.check_status()
    assert abs(loss.item() - ref.item()) < 2e-3
    ge = dict(eager.named_parameters())
    for k, p in native.named_parameters():
        g = p.grad
        if "w_gate_up" in k:
            gref = torch.cat((ge[k.replace("w_gate_up", "gate_proj")].grad, ge[k.replace("w_gate_up", "up_proj")].grad))
        elif "w_down" in k:
            gref = ge[k.replace("w_down", "down_proj")].grad
        else:
            gref = ge[k].grad
        # Error budget from the arithmetic: activations and gradients are rounded to bf16 (unit round-off 2^-8) at
        # every kernel boundary and the roundings of a path add up roughly in quadrature.  The head tensors sit two
        # roundings from the loss, everything below them behind a dozen or more: 2 and 4 units of 2^-8 (observed
        # 1.0 - 1.4 and 2.0 - 3.0 units).
        rel = (g - gref).norm() / (gref.norm() + 1e-12)
        units = 2 if k in ("lm_head.weight", "final_norm.weight") else 4
        assert rel.item() < units * 2.0 ** -8, (k, rel.item())


def test_training_reduces_loss_and_fsdp_single_gpu_matches_plain():
    from llm_systems_from_scratch_b200.ops import native as nat
    from llm_systems_from_scratch_b200.optim import FusedAdamW
    from llm_systems_from_scratch_b200.parallel import FSDP
    _, a = _models()
    _, b = _models()
    fb = FSDP(b)
    oa = FusedAdamW(a.parameters(), lr=1e-3, weight_decay=0.1)
    ob = FusedAdamW(fb.parameters(), lr=1e-3, weight_decay=0.1)
    x = torch.randint(0, CFG["vocab_size"], (4, 256), device="cuda")
    y = torch.randint(0, CFG["vocab_size"], (4, 256), device="cuda")
    la, lb = [], []
    for _ in range(5):
        l1 = a.loss(x, y)
        l1.backward()
        oa.set_grad_scale(a.engine().provider.arena.clip_coef(1.0))
        oa.step()
        l2 = fb.loss(x, y)
        l2.backward()
        fb.finish_gradient_synchronization()
        ob.set_grad_scale(fb.shard_arena.clip_coef(1.0))
        ob.step()
        la.append(l1.item())
        lb.append(l2.item())
    nat.check_status()
    assert la[-1] < la[0] - 0.05, la
    assert max(abs(p - q) for p, q in zip(la, lb)) < 1e-3, (la, lb)


def test_activation_checkpointing_matches():
    _, a = _models()
    _, b = _models()
    b.activation_checkpointing = True
    x = torch.randint(0, CFG["vocab_size"], (2, 256), device="cuda")
    y = torch.randint(0, CFG["vocab_size"], (2, 256), device="cuda")
    a.loss(x, y).backward()
    b.loss(x, y).backward()
    for (k, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p.grad, q.grad), k


def test_smoke_entry():
    import __graft_entry__
    __graft_entry__.smoke()


def test_training_is_bitwise_reproducible():
    """Every reduction on the training path has a fixed order (no float atomics), so two runs from the same seed end
    with identical parameters; a race between kernels or streams would show up here as a difference."""
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.ops import native as nat
    from llm_systems_from_scratch_b200.optim import FusedAdamW
    from llm_systems_from_scratch_b200.parallel import FSDP
    cfg = dict(vocab_size=1003, context_length=512, d_model=512, num_layers=3, num_heads=4, d_ff=1408, rope_theta=10000.0)

    def run():
        torch.manual_seed(0)
        model = TransformerLM(**cfg, use_flash_attn=True, use_custom_triton=True).cuda()
        wrapped = FSDP(model)
        opt = FusedAdamW(wrapped.parameters(), lr=1e-3, weight_decay=0.1)
        g = torch.Generator(device="cuda").manual_seed(1)
        losses = []
        for _ in range(4):
            x = torch.randint(0, cfg["vocab_size"], (4, 512), device="cuda", generator=g)   # 2048 rows: CTA-pair GEMMs
            y = torch.randint(0, cfg["vocab_size"], (4, 512), device="cuda", generator=g)
            loss = wrapped.loss(x, y)
            loss.backward()
            wrapped.finish_gradient_synchronization()
            opt.set_grad_scale(wrapped.shard_arena.clip_coef(1.0))
            opt.step()
            losses.append(loss.item())
        nat.check_status()
        return losses, [p.detach().clone() for p in wrapped.parameters()]

    l1, p1 = run()
    l2, p2 = run()
    assert l1 == l2
    assert all(torch.equal(a, b) for a, b in zip(p1, p2))
