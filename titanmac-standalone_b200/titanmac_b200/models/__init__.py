from .titanmac import TitanMAC

__all__ = ["TitanMAC"]
