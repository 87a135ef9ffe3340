"""Model families built on the fused ops (Llama-shaped tensor-parallel decoders)."""
