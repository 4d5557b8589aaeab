"""sm_100a implementations behind the registries of ``embodiinfer_b200.layers``."""
