"""Comparison helpers with the names and defaults of the reference's ``daceml.testing`` (``daceml/testing/utils.py:33-77``)."""
import numpy as np
import torch


def tensors_close(name, expected, result, rtol=1e-5, atol=1e-5):
    def to_numpy(x):
        return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)

    np.testing.assert_allclose(to_numpy(result), to_numpy(expected), rtol=rtol, atol=atol, err_msg=f"{name} not close")


def torch_tensors_close(name, torch_v, dace_v, rtol=1e-5, atol=1e-4):
    """Assert that the two torch tensors are close and on the same device."""
    assert torch_v.device == dace_v.device, "Tensors are on different devices"
    np.testing.assert_allclose(torch_v.detach().float().cpu().numpy(), dace_v.detach().float().cpu().numpy(), rtol=rtol, atol=atol,
                               err_msg=f"{name} not close")


def copy_to_gpu(gpu: bool, tensor):
    return tensor.cuda() if gpu else tensor
