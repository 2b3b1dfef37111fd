"""CPU oracle for the routed-expert MoE path (test infrastructure, never imported by the package)."""
