"""CPU oracle (test infrastructure only): see oracle/wein_oracle.c."""
