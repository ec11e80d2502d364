"""``cupy.cuda.device.Device().compute_capability`` -> ``"100"`` on a B200."""
import torch


class Device:
    def __init__(self, device=None):
        self.id = torch.cuda.current_device() if device is None else int(device)

    @property
    def compute_capability(self) -> str:
        major, minor = torch.cuda.get_device_capability(self.id)
        return f"{major}{minor}"
