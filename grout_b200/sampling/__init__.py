from .device import DeviceSampler
from .draws import DrawStream
from .host import HostSampler, choose_one
from .params import SamplingParams

__all__ = ["DeviceSampler", "DrawStream", "HostSampler", "choose_one", "SamplingParams"]
