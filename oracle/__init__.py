"""CPU oracle for the parity tests. Test infrastructure only: nothing under tensorrt_b200/ imports it."""
