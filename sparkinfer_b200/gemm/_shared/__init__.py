"""Host code shared by the linear ops."""
