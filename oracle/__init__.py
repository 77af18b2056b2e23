"""CPU oracle of the GCT streaming attention path.  Test infrastructure, not product code:
only the tests, the smoke check and the CPU-baseline legs of the benchmark import it."""
