"""CPU oracle of the dense-contraction path.  TEST INFRASTRUCTURE ONLY: nothing under
tritonix_b200/ may import it; only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline
legs do."""
