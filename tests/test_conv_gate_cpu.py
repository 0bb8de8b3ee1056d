"""The convolutional gate falls back to the PyTorch layers wherever the fused kernels do not apply."""
import torch
from torch import nn

from dice_embeddings_b200.models import initialize_model
from dice_embeddings_b200.ops import conv_gate


def test_cpu_tensors_are_not_claimed_by_the_fused_path():
    conv, bn = nn.Conv2d(1, 2, 3, padding=1), nn.BatchNorm2d(2)
    assert not conv_gate.supported(torch.randn(8, 64), conv, bn, 4, 16)


def test_conv_models_give_the_same_scores_with_the_switch_on_and_off_on_cpu():
    torch.manual_seed(0)
    for name, d in (("ConEx", 16), ("AConvQ", 32), ("ConvO", 32)):
        args = dict(model=name, embedding_dim=d, num_entities=50, num_relations=5, optim="Adam", learning_rate=0.01,
                    scoring_technique="KvsAll", num_of_output_channels=2, kernel_size=3)
        model, _ = initialize_model(args)
        model.eval()
        x = torch.stack((torch.randint(0, 50, (12,)), torch.randint(0, 5, (12,))), 1)
        with torch.no_grad():
            on = model.forward_k_vs_all(x)
            model.fused_conv_gate = False
            off = model.forward_k_vs_all(x)
        assert torch.equal(on, off)
