"""Inference: paged KV cache bookkeeping, continuous-batching scheduler, generation engine and an OpenAI-compatible server."""
