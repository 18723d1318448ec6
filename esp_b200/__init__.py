"""esp_b200: a small, whole generation library for one GPU."""
