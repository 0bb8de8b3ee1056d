"""Fused convolution + batch normalisation + ReLU of the convolutional gate models against the PyTorch layers."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("CUDA device required", allow_module_level=True)

from dice_embeddings_b200.models import initialize_model
from dice_embeddings_b200.ops import conv_gate

DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _fp32_convolutions():
    """The oracle is the PyTorch layers in full fp32 (cuDNN convolutions default to TF32)."""
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cudnn.allow_tf32 = old


def _layers(C):
    torch.manual_seed(3)
    conv = nn.Conv2d(1, C, 3, padding=1).to(DEV)
    bn = nn.BatchNorm2d(C).to(DEV)
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.uniform_(-0.3, 0.3)
        bn.running_mean.uniform_(-0.2, 0.2)
        bn.running_var.uniform_(0.5, 1.5)
    return conv, bn


def _torch_path(x, conv, bn, H, W):
    return torch.relu(bn(conv(x.view(-1, 1, H, W)))).reshape(x.shape[0], -1)


@pytest.mark.parametrize("B,H,W,C", [(37, 4, 16, 2), (300, 8, 16, 4), (1000, 16, 16, 8), (64, 4, 128, 3)])
@pytest.mark.parametrize("training", [True, False])
def test_features_and_gradients_equal_the_layers(B, H, W, C, training):
    import copy
    conv, bn = _layers(C)
    conv2, bn2 = copy.deepcopy(conv), copy.deepcopy(bn)
    for m in (bn, bn2):
        m.train(training)
    torch.manual_seed(B)
    x1 = torch.randn(B, H * W, device=DEV, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_(True)
    assert conv_gate.supported(x1, conv, bn, H, W)
    f1 = conv_gate.conv_gate_features(x1, conv, bn, H, W)
    f2 = _torch_path(x2, conv2, bn2, H, W)
    assert torch.allclose(f1, f2, atol=2e-5, rtol=1e-4)
    assert torch.allclose(bn.running_mean, bn2.running_mean, atol=1e-6)
    assert torch.allclose(bn.running_var, bn2.running_var, atol=1e-5, rtol=1e-5)
    if training:
        assert int(bn.num_batches_tracked) == int(bn2.num_batches_tracked) == 1
    g = torch.randn_like(f1)
    f1.backward(g)
    f2.backward(g)

    def close(a, b, what, tol=2e-4):
        scale = b.abs().max().clamp_min(1e-6)
        assert (a - b).abs().max() <= tol * scale + 1e-6, (what, float((a - b).abs().max()), float(scale))

    # An output within rounding distance of zero may open the ReLU in one implementation and close it in the other;
    # each such position changes the nine image gradients under its window and moves the reduced gradients a little.
    bad = (x1.grad - x2.grad).abs() > 2e-4 * x2.grad.abs().max() + 1e-6
    assert int(bad.sum()) <= 27, int(bad.sum())
    close(conv.weight.grad, conv2.weight.grad, "weight", 5e-3)
    if not training:   # with batch statistics the bias gradient is a difference of equal sums: compare absolutely
        close(conv.bias.grad, conv2.bias.grad, "bias", 5e-3)
    else:
        assert conv.bias.grad.abs().max() <= 1e-5 * g.abs().sum()
    close(bn.weight.grad, bn2.weight.grad, "gamma", 5e-3)
    close(bn.bias.grad, bn2.bias.grad, "beta", 5e-3)


def test_unsupported_shapes_are_reported():
    conv, bn = _layers(16)
    x = torch.randn(8, 64, device=DEV)
    assert not conv_gate.supported(x, conv, bn, 4, 16)           # more than 8 channels
    conv5 = nn.Conv2d(1, 2, 5, padding=1).to(DEV)
    assert not conv_gate.supported(x, conv5, nn.BatchNorm2d(2).to(DEV), 4, 16)
    assert not conv_gate.supported(x.cpu(), *_layers(2), 4, 16)


@pytest.mark.parametrize("name,D", [("ConEx", 32), ("AConEx", 32), ("ConvQ", 64), ("AConvQ", 64), ("ConvO", 64),
                                    ("AConvO", 64)])
def test_models_train_identically_with_and_without_the_fused_gate(name, D):
    torch.manual_seed(5)
    args = dict(model=name, embedding_dim=D, num_entities=200, num_relations=9, optim="Adam", learning_rate=0.01,
                scoring_technique="KvsAll", num_of_output_channels=2, kernel_size=3)
    m1, _ = initialize_model(dict(args))
    m2, _ = initialize_model(dict(args))
    m2.load_state_dict(m1.state_dict())
    m1.to(DEV), m2.to(DEV)
    m2.fused_conv_gate = False
    x = torch.stack((torch.randint(0, 200, (96,)), torch.randint(0, 9, (96,))), 1).to(DEV)
    y = (torch.rand(96, 200, device=DEV) < 0.05).float()
    for m in (m1, m2):
        m.train()
        loss = torch.nn.functional.binary_cross_entropy_with_logits(m.forward_k_vs_all(x), y)
        loss.backward()
        m.last_loss = float(loss.detach())
    assert abs(m1.last_loss - m2.last_loss) < 1e-5
    for (n1, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        if p2.grad is None:
            assert p1.grad is None, n1
            continue
        scale = p2.grad.abs().max().clamp_min(1e-7)
        assert (p1.grad - p2.grad).abs().max() <= 1e-3 * scale + 1e-7, n1
    m1.eval(), m2.eval()
    with torch.no_grad():
        assert torch.allclose(m1.forward_k_vs_all(x), m2.forward_k_vs_all(x), atol=1e-4, rtol=1e-4)


def test_fused_gate_is_faster_than_the_layers():
    torch.backends.cudnn.allow_tf32 = True   # the library's default: the comparison a user would see
    B, H, W, C = 4096, 4, 128, 8
    conv, bn = _layers(C)
    x = torch.randn(B, H * W, device=DEV, requires_grad=True)

    def run(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / 10

    def fused():
        conv_gate.conv_gate_features(x, conv, bn, H, W).sum().backward()

    def layers():
        _torch_path(x, conv, bn, H, W).sum().backward()

    t_fused, t_layers = run(fused), run(layers)
    print(f"conv gate fwd+bwd B={B} {H}x{W} C={C}: fused {t_fused:.3f} ms, layers {t_layers:.3f} ms")
    assert t_fused < t_layers
