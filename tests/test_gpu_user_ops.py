"""User CUDA kernels registered with make_torch_op_from_mojo, run eagerly and inside graphs compiled
with mojo_backend, against eager PyTorch on the CPU (the reference's tests/test_compiler.py:766-935
with its Mojo kernels replaced by the CUDA kernels of tests/dummy_cuda_kernels)."""

from pathlib import Path

import pytest
import torch
from torch._dynamo import mark_dynamic

from torch_mojo_backend import make_torch_op_from_mojo, mojo_backend

pytestmark = pytest.mark.gpu
KERNELS = Path(__file__).parent / "dummy_cuda_kernels"


def allocate_outputs_grayscale(pic: torch.Tensor) -> torch.Tensor:
    return pic.new_empty(pic.shape[:-1], dtype=torch.float32)


def grayscale_eager(pic):
    pic = pic.to(dtype=torch.float32)
    r, g, b = pic[:, :, 0], pic[:, :, 1], pic[:, :, 2]
    return torch.clamp(0.21 * r + 0.71 * g + 0.07 * b, max=255)


def allocate_outputs_grayscale_multi(pic: torch.Tensor, noise: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return tuple(pic.new_empty(noise.shape, dtype=torch.float32) for _ in range(2))


def grayscale_multi_eager(pic, noise):
    pic = pic.to(dtype=torch.float32)
    r, g, b = pic[:, :, 0] + noise, pic[:, :, 1] + noise, pic[:, :, 2] + noise
    return torch.clamp(0.21 * r + 0.71 * g + 0.07 * b, max=255), r


def picture(h=224, w=224, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (h, w, 3), generator=g, dtype=torch.uint8)


def test_user_op_eager_and_in_a_compiled_graph():
    gray = make_torch_op_from_mojo(KERNELS, "grayscale", allocate_outputs_grayscale)
    img = picture()
    torch.testing.assert_close(gray(img.cuda()).cpu(), grayscale_eager(img))
    # a strided view goes through untouched: the kernel gets the strides
    wide = picture(224, 448, 1)
    torch.testing.assert_close(gray(wide.cuda()[:, ::2]).cpu(), grayscale_eager(wide[:, ::2]))
    assert gray(img.cuda()[:0]).shape == (0, 224)

    def graph(x):
        return gray(x + 8) - 16

    def graph_eager(x):
        return grayscale_eager(x + 8) - 16

    compiled = torch.compile(graph, backend=mojo_backend, fullgraph=True)
    torch.testing.assert_close(compiled(img.cuda()).cpu(), graph_eager(img))
    torch.testing.assert_close(compiled(img.cuda()).cpu(), graph_eager(img))  # the cached plan
    explanation = torch._dynamo.explain(graph)(img.cuda())
    assert explanation.graph_break_count == 0 and explanation.graph_count == 1


def test_user_op_with_two_outputs():
    multi = make_torch_op_from_mojo(KERNELS, "grayscale_multi", allocate_outputs_grayscale_multi)
    img = picture(seed=2)
    noise = torch.randint(0, 2, (224, 224), generator=torch.Generator().manual_seed(3)).to(torch.uint8)
    x1, x2 = multi(img.cuda(), noise.cuda())
    y1, y2 = grayscale_multi_eager(img, noise)
    torch.testing.assert_close(x1.cpu(), y1)
    torch.testing.assert_close(x2.cpu(), y2)

    def graph(x, n):
        y1, y2 = multi(x + 8, n)
        return y1 - 16, y2 + 3

    def graph_eager(x, n):
        y1, y2 = grayscale_multi_eager(x + 8, n)
        return y1 - 16, y2 + 3

    compiled = torch.compile(graph, backend=mojo_backend, fullgraph=True)
    z1, z2 = compiled(img.cuda(), noise.cuda())
    w1, w2 = graph_eager(img, noise)
    torch.testing.assert_close(z1.cpu(), w1)
    torch.testing.assert_close(z2.cpu(), w2)
    explanation = torch._dynamo.explain(graph)(img.cuda(), noise.cuda())
    assert explanation.graph_break_count == 0 and explanation.graph_count == 1


def test_user_op_with_dynamic_dims():
    multi = make_torch_op_from_mojo(KERNELS, "grayscale_multi", allocate_outputs_grayscale_multi)

    def graph(x, n):
        y1, y2 = multi(x + 8, n)
        return y1 - 16, y2 + 3

    compiled = torch.compile(graph, backend=mojo_backend, fullgraph=True)
    for h, w in ((224, 224), (96, 160), (33, 7)):
        img = picture(h, w, seed=h)
        noise = torch.randint(0, 2, (h, w), generator=torch.Generator().manual_seed(w)).to(torch.uint8)
        a, b = img.cuda(), noise.cuda()
        for t in (a, b):
            mark_dynamic(t, 0)
            mark_dynamic(t, 1)
        z1, z2 = compiled(a, b)
        y1, y2 = grayscale_multi_eager(img + 8, noise)
        torch.testing.assert_close(z1.cpu(), y1 - 16)
        torch.testing.assert_close(z2.cpu(), y2 + 3)


def test_user_op_status_is_raised():
    gray = make_torch_op_from_mojo(KERNELS, "grayscale", allocate_outputs_grayscale)
    with pytest.raises(RuntimeError, match="returned status 2"):
        gray(torch.zeros(4, 4, 4, dtype=torch.uint8, device="cuda"))  # four channels: the kernel refuses
