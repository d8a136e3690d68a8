"""Symmetric memory and groups."""
from . import symm_mem
from .symm_mem import EmuWorld, GroupInfo, SymmHandle, resolve_group

__all__ = ["symm_mem", "EmuWorld", "GroupInfo", "SymmHandle", "resolve_group"]
