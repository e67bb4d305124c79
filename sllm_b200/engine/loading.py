"""From a model folder to a model on the device: config.json chooses the
architecture through the registry, the plan builds the parts, the loader binds
the folder's tensors by name."""

from __future__ import annotations

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.registry import load_config
from ..models.causal_lm import CausalLM
from ..weights.loader import load_into

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {name!r}") from None


SLACK_BYTES = 512 << 20      # left free beside the weights: the cache and the step's buffers need room too


def resident_bytes(model: CausalLM) -> int:
    """Device bytes the model's tensors will take once bound (from its tensor specs, in the dtype each
    is kept in: matrices and tables in the compute dtype, gains and biases in float32)."""
    itemsize = torch.empty((), dtype=model.dtype).element_size()
    total = 0
    for s in model.tensor_specs():
        n = 1
        for d in s.shape:
            n *= int(d)
        total += n * (4 if s.role in ("gain", "bias") else itemsize)
    return total


def check_device_memory(model: CausalLM) -> None:
    """Refuse to start an upload that cannot fit: a clear error before the first copy instead of an
    out-of-memory fault in the middle of it (the reference guards its resident upload the same way,
    kernels/device_decode.py:100-114)."""
    dev = torch.device(model.device)
    if dev.type != "cuda":
        return
    need = resident_bytes(model)
    free, total = torch.cuda.mem_get_info(dev)
    if free < need + SLACK_BYTES:
        raise MemoryError(f"the model's weights take {need / 2**30:.2f} GiB on {dev}; {free / 2**30:.2f} GiB of "
                          f"{total / 2**30:.2f} GiB are free and {SLACK_BYTES / 2**30:.2f} GiB must stay free beside them")


def build_model(model_dir: str, dtype="bfloat16", device="cuda:0", *, progress=None):
    """(model, typed config) of the folder, weights bound."""
    arch, cfg = load_config(model_dir)
    model = CausalLM(arch.plan(cfg), dtype=parse_dtype(dtype), device=device)
    check_device_memory(model)
    load_into(model, model_dir, progress=progress)
    return model, cfg


def build_random_model(config: dict, seed: int, dtype="bfloat16", device="cuda:0", *, std: float = 0.02,
                       gain_std: float = 0.0):
    """A model of ``config`` (config.json's keys) with weights drawn on the device, one
    tensor at a time, without a model folder: for sizes whose folder would take minutes to
    write and read.  (model, typed config)."""
    from ..config.registry import architecture_of
    arch = architecture_of(config)
    cfg = arch.config_cls.from_dict(config)
    dt = parse_dtype(dtype)
    model = CausalLM(arch.plan(cfg), dtype=dt, device=device)
    check_device_memory(model)
    specs = {s.name: s for s in model.tensor_specs()}
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)

    def fetch(name):
        s = specs[name]
        if s.role == "gain":
            t = torch.ones(s.shape, dtype=torch.float32, device=device)
            if gain_std:
                t += gain_std * torch.randn(s.shape, generator=gen, device=device)
            return t
        t = torch.empty(s.shape, dtype=dt if s.role != "bias" else torch.float32, device=device)
        t.normal_(0.0, std, generator=gen)
        return t

    model.bind(fetch)
    return model, cfg
