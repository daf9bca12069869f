"""CPU parity oracle for the GrainGEMM hot path. Test infrastructure only."""
