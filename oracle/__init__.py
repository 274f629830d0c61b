"""Test infrastructure: CPU oracle of the attention path (see attn_oracle.h). Not part of the product."""
