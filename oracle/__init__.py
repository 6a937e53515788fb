"""CPU oracle of the reference sampler: test infrastructure only, never imported by the package."""
