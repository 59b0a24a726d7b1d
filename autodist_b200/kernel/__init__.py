"""Transformation passes that turn (captured graph, compiled strategy) into an executable plan."""
