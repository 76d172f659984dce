from . import functional
from .modules import *  # noqa: F401,F403
