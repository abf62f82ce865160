"""LayerwiseGradientScaler inside training loops (cases of the reference's tests/optim/test_layerwise_gradient_scaler.py with
synthetic data in place of its downloaded sets): a feed-forward classifier and a small convolutional network trained with and
without per-layer factors end with the same gradients and weights; under CPU autocast; layers that are not named are left
alone; an empty table is a no-op."""
import pytest
import torch
from torch import nn

from fairscale_b200.optim import LayerwiseGradientScaler


class _FeedForward(nn.Module):
    def __init__(self, inputs=2, hidden=10):
        super().__init__()
        torch.manual_seed(7)
        self.fc1, self.relu1 = nn.Linear(inputs, hidden), nn.ReLU()
        self.fc2, self.relu2 = nn.Linear(hidden, hidden), nn.ReLU()
        self.fc3, self.sigmoid, self.identity = nn.Linear(hidden, 1), nn.Sigmoid(), nn.Identity()

    def forward(self, x):
        return self.identity(self.sigmoid(self.fc3(self.relu2(self.fc2(self.relu1(self.fc1(x)))))))


class _ConvNet(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(24)
        self.conv1, self.relu1, self.pool1 = nn.Conv2d(3, 6, 5), nn.ReLU(), nn.MaxPool2d(2, 2)
        self.conv2, self.relu2, self.pool2 = nn.Conv2d(6, 16, 5), nn.ReLU(), nn.MaxPool2d(2, 2)
        self.fc1, self.relu3 = nn.Linear(16 * 5 * 5, 120), nn.ReLU()
        self.fc2, self.relu4 = nn.Linear(120, 84), nn.ReLU()
        self.fc3, self.identity = nn.Linear(84, 10), nn.Identity()

    def forward(self, x):
        x = self.pool2(self.relu2(self.conv2(self.pool1(self.relu1(self.conv1(x))))))
        x = torch.flatten(x, 1)
        return self.identity(self.fc3(self.relu4(self.fc2(self.relu3(self.fc1(x))))))


def _blobs():
    g = torch.Generator().manual_seed(11)
    centres = torch.tensor([[2.0, 2.0], [-2.0, -2.0], [2.0, -2.0], [-2.0, 2.0]])
    which = torch.randint(0, 4, (40,), generator=g)
    x = centres[which] + 1.5 * torch.randn(40, 2, generator=g)
    return x, (which != 0).float()


def _train_classifier(table, autocast):
    model = _FeedForward()
    opt = torch.optim.SGD(model.parameters(), lr=0.001)
    x, y = _blobs()
    scaler = LayerwiseGradientScaler(model, table)
    for _ in range(2):
        opt.zero_grad()
        scaler.scale()
        with torch.autocast("cpu", dtype=torch.bfloat16, enabled=autocast):
            loss = nn.functional.binary_cross_entropy_with_logits(model(x).squeeze().float(), y)
        loss.backward()
        scaler.unscale()
        scaler.step(opt)
    return model


@pytest.mark.parametrize("autocast", [False, True])
def test_feed_forward_classifier_trains_the_same_with_and_without_factors(autocast):
    plain = _train_classifier({}, autocast)
    scaled = _train_classifier({"fc1": 1024, "fc2": 512, "fc3": 1024}, autocast)
    tol = dict(atol=1e-3, rtol=5e-2) if autocast else dict(atol=1e-8, rtol=1e-5)  # bf16 rounds the scaled values differently
    for a, b in zip(plain.parameters(), scaled.parameters()):
        torch.testing.assert_close(b.grad, a.grad, **tol)
        torch.testing.assert_close(b, a, **tol)


def _train_convnet(table):
    model = _ConvNet()
    opt = torch.optim.SGD(model.parameters(), lr=0.001, momentum=0.9)
    g = torch.Generator().manual_seed(10)
    scaler = LayerwiseGradientScaler(model, table)
    for _ in range(3):
        images, labels = torch.randn(16, 3, 32, 32, generator=g), torch.randint(0, 10, (16,), generator=g)
        opt.zero_grad()
        scaler.scale()
        nn.functional.cross_entropy(model(images), labels).backward()
        scaler.unscale()
        scaler.step(opt)
    return model, scaler


def test_convolutional_network_trains_the_same_with_and_without_factors():
    plain, _ = _train_convnet({})
    scaled, scaler = _train_convnet({"conv1": 128, "conv2": 256, "fc1": 512, "fc2": 1024, "fc3": 8192})
    for a, b in zip(plain.parameters(), scaled.parameters()):
        torch.testing.assert_close(b.grad, a.grad, atol=1e-6, rtol=1e-4)
        torch.testing.assert_close(b, a, atol=1e-6, rtol=1e-4)
    scaled_layers = [info for info in scaler.get_layer_info() if info.scale_layer]
    assert [info.layer_name for info in scaled_layers] == ["conv1", "conv2", "fc1", "fc2", "fc3"]
    assert all(info.scaling_factor >= 128 for info in scaled_layers)


def test_layers_that_are_not_named_are_left_alone():
    model = _FeedForward()
    scaler = LayerwiseGradientScaler(model, {"fc2": 64.0})
    x, y = _blobs()
    scaler.scale()
    nn.functional.binary_cross_entropy_with_logits(model(x).squeeze(), y).backward()
    scaled_grad = model.fc2.weight.grad.clone()
    other_grad = model.fc3.weight.grad.clone()
    scaler.unscale()
    torch.testing.assert_close(model.fc2.weight.grad * 64.0, scaled_grad)
    assert torch.equal(model.fc3.weight.grad, other_grad)  # never multiplied, never divided
    infos = {info.layer_name: info for info in scaler.get_layer_info()}
    assert infos["fc2"].scale_layer and not infos["fc1"].scale_layer and not infos["fc3"].scale_layer
