"""The sampler CLI keeps the reference's flags (sample.py:20-33 of the reference)."""
import inspect
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sample_main_has_the_reference_flags():
    sys.path.insert(0, ROOT)
    import importlib

    sample = importlib.import_module("sample")
    params = inspect.signature(sample.main).parameters
    for name, default in [
        ("prompt", None), ("negative_prompt", ""), ("seed", 42), ("guidance_scale", 5.0), ("num_inference_steps", 50),
        ("width", 1024), ("height", 1024), ("compile_unet", False), ("fp16_acc_matmul", False), ("patch_parallelism", True),
        ("distrifusion_warmup_steps", 4), ("verbose", False),
    ]:
        assert name in params, name
        if default is not None:
            assert params[name].default == default, name


def test_config_defaults_match_the_reference():
    from basedxl_b200.utils import BasedXLConfig
    import torch

    c = BasedXLConfig(device_type="cpu")
    assert (c.dtype, c.fp16_acc_matmul, c.patch_parallelism, c.compile_unet, c.width, c.height, c.use_cfg, c.warmup_steps,
            c.comm_checkpoint, c.verbose) == (torch.float16, False, False, False, 1024, 1024, True, 4, 60, False)
    assert (c.rank, c.world_size, c.n_device_per_batch, c.batch_group, c.split_group) == (0, 1, 1, None, None)
    assert c.batch_idx() == 1 and c.split_idx() == 0  # the reference's single-device values (basedxl/utils.py:62-73)
    # the rank -> (CFG half, strip) map of an 8-GPU run
    c.world_size, c.n_device_per_batch = 8, 4
    assert [c.batch_idx(r) for r in range(8)] == [0, 0, 0, 0, 1, 1, 1, 1]
    assert [c.split_idx(r) for r in range(8)] == [0, 1, 2, 3, 0, 1, 2, 3]
