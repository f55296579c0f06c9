"""CPU oracle for the q4_0 path: test infrastructure only.  The product never imports this."""
