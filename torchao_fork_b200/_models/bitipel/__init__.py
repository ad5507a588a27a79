from .model import Bitipel, BitipelArgs, bitipel_configs  # noqa: F401
