"""Host-side glue shared by the operator layer (streams)."""
