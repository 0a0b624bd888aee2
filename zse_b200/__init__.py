"""zse_b200 — a Blackwell (sm_100a) LLM inference engine that serves ``.zse`` models."""
__version__ = "0.1.0"
