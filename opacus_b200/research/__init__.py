"""Research add-ons that build on the DP optimizers (not part of the stable API)."""
