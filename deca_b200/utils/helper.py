"""GPU detection (the part of the reference's src/utils/helper.py:51-99 the hot path uses)."""

from ..arch.B200 import B200


def byte_size(dtype: str) -> int:
    return {"float32": 4, "float16": 2, "bfloat16": 2}[dtype]


class GPUDetector:
    """Maps the visible device's name to its hardware model."""

    GPU_MODEL_MAP = {
        "NVIDIA B200": B200,
    }

    @classmethod
    def detect_gpu(cls, verbose: bool):
        """Returns the Arch class of device 0; prints the reason and exits(-1) when there is
        no device or its model is unknown (the reference's behaviour, helper.py:78-89)."""
        try:
            import torch

            if not torch.cuda.is_available():
                raise RuntimeError("no CUDA device is visible")
            name = torch.cuda.get_device_name(0)
            if verbose:
                print(f"Detected GPU: {name}")
            if name in cls.GPU_MODEL_MAP:
                return cls.GPU_MODEL_MAP[name]
            raise NotImplementedError(
                f"Unsupported GPU model: {name}; this build only targets {list(cls.GPU_MODEL_MAP)}."
            )
        except Exception as e:  # noqa: BLE001
            print(f"GPU detection failed: {e}")
            raise SystemExit(-1)

    @classmethod
    def create_gpu_instance(cls, verbose=True):
        gpu = cls.detect_gpu(verbose=verbose)()
        if hasattr(gpu, "configure_device"):
            gpu.configure_device(0)
        return gpu
