from .options import GenOptions, OptionError, OPTION_TABLE, render_help
from .sampler import DeviceSampler, sampler_state

__all__ = ["GenOptions", "OptionError", "OPTION_TABLE", "render_help", "DeviceSampler", "sampler_state"]
