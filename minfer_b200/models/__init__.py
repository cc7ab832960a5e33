"""Architectures that ship with the library, registered under their config.json names."""
from ..config.bedarax import ARCHITECTURE as BEDARAX, BedaraxConfig
from ..config.budanex import ARCHITECTURE as BUDANEX, BudanexConfig
from ..config.furitar import ARCHITECTURE as FURITAR, FuritarConfig
from ..config.qwen2 import ARCHITECTURE as QWEN2, Qwen2Config
from ..config.zanelorn import ARCHITECTURE as ZANELORN, ZanelornConfig
from ..registry import register_architecture

register_architecture(QWEN2, Qwen2Config.from_dict, replace=True)
register_architecture(FURITAR, FuritarConfig.from_dict, replace=True)
register_architecture(BUDANEX, BudanexConfig.from_dict, replace=True)
register_architecture(BEDARAX, BedaraxConfig.from_dict, replace=True)
register_architecture(ZANELORN, ZanelornConfig.from_dict, replace=True)
