{
  global:
    plaidml_*;
    pmlb_*;
  local:
    *;
};
