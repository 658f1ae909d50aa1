"""Architectures register themselves on import."""
from . import gpt2  # noqa: F401
from . import sovozen  # noqa: F401
from . import gokezen  # noqa: F401
from . import rakarax  # noqa: F401
from . import bosalix  # noqa: F401
