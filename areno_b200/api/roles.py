"""Auxiliary model roles (reference / critic / reward) named by algorithms and owned by the backend."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class ModelRole:
    name: str
    path: str
    trainable: bool
    optimizer_lr: float | None = None


class MissingRoleCapability(RuntimeError):
    """The backend cannot execute a role operation an algorithm needs."""
