from .control_flow import fori_loop  # noqa: F401
from .knob import knob  # noqa: F401
