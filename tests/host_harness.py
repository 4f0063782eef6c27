"""A runner for host-logic tests: the package's step function, cache manager and decoder
assembly, on the CPU, with every CUDA kernel replaced by its restatement in
``kernel_refs``.  It exercises packing, block tables, page reuse and the layer order
without a GPU; the kernels themselves are tested on the GPU."""

from __future__ import annotations

import torch

from emberserve_b200.engine.runner import ModelRunner


class HostRunner(ModelRunner):
    _require_cuda = False


def host_runner(model_dir, dtype=torch.float32, **kw) -> HostRunner:
    return HostRunner.from_dir(model_dir, dtype, device="cpu", **kw)
