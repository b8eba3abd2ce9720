"""CPU oracle (test infrastructure).  See illatio_oracle.c."""
