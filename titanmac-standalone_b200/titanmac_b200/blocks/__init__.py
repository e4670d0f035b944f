from .titan_block import MLPBlock, RMSNorm, TitanBlock

__all__ = ["MLPBlock", "RMSNorm", "TitanBlock"]
