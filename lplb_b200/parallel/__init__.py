"""Cross-GPU plumbing: bootstrap of the peer-memory statistics exchange and its CPU protocol model."""

from .exchange import open_peer_exchange

__all__ = ["open_peer_exchange"]
