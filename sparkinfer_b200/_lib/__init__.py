"""Host-side support code shared by the op packages (stdlib + torch only)."""
