"""Drop-in counterparts of UniQL's `quantize` package modules that sit on the inference hot path."""
