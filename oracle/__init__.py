"""CPU oracle package (test infrastructure only; never imported by ``lucid_b200``)."""
