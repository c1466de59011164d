"""Small offline tools (quality gates on saved logits and token lists)."""
