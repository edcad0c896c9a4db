"""QuickGELU on the CUDA entry point; same class as triteia/python/capi/activations.py:5-24."""
import torch

from .. import triteia_cuda


class QuickGELU:
    def __init__(self):
        self.op = triteia_cuda.gelu_quick

    def forward_native(self, x: torch.Tensor) -> torch.Tensor:
        """PyTorch statement of forward()."""
        return x * torch.sigmoid(1.702 * x)

    def forward_cuda(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        self.op(out, x)
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_cuda(x)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward(x)
