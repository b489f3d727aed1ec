from . import build, ops
