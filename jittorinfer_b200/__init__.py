"""jittorinfer_b200 — a Blackwell (sm_100a) native LLM inference engine for the DeepSeek-V2 family."""
__version__ = "0.1.0"
