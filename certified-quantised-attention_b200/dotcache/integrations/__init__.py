"""Model adapters over the certified decode-attention path."""
