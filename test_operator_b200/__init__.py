"""B200-native sparse MLA attention backward (drop-in for the reference's `mla_bwd` operator)."""
