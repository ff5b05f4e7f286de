"""teramoe_b200: Blackwell-native expert-parallel MoE training library."""
