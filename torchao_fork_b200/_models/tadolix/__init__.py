from .model import Tadolix, TadolixArgs, tadolix_configs  # noqa: F401
