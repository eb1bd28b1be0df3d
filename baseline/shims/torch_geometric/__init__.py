"""Minimal stand-in for the handful of ``torch_geometric.utils`` helpers the reference imports."""
from . import utils  # noqa: F401
