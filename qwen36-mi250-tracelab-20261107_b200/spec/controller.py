"""MTP speculative decoding controller (filled in by spec/mtp_chain)."""

from __future__ import annotations


class SpecController:
    """Placeholder wiring: no speculation until the chain verify path is enabled."""

    def __init__(self, engine) -> None:
        self.engine = engine

    def after_prefill(self, gens, spans, batch, hidden) -> None:
        return None

    def first_drafts(self, gens) -> None:
        return None

    def step(self, running) -> bool:
        return False

    def settle(self, gen) -> None:
        return None
