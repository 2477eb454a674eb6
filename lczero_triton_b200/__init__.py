"""B200-native forward pass for Lc0 BT4-style transformer networks."""
