from .sampler import DeviceSelector
