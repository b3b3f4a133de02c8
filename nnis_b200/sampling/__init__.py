from .config import SAMPLING_POLICY_VERSION, SamplingConfig, SamplingError
from .host import HostLogitSampler, SplitMix64

__all__ = ["SAMPLING_POLICY_VERSION", "SamplingConfig", "SamplingError", "HostLogitSampler",
           "SplitMix64"]
