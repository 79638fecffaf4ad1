"""Experimental algorithms: sub-packages here are imported on demand and may call
``areno_b200.api.algorithms.register_algorithm``."""
