"""CPU oracle for the WKV7 recurrence: test infrastructure, never a product path."""
