"""CPU oracle for the fused-turboquant hot path (test infrastructure only)."""
