from .adopt import ADOPT

__all__ = ["ADOPT"]
