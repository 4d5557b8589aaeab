"""CPU restatement of the reference's quantised-Linear arithmetic: test infrastructure only."""
