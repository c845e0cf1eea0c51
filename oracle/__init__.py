"""CPU oracle (test infrastructure).  Only tests, the smoke check and the benchmark's CPU legs import this."""
