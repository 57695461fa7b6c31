/* TEST INFRASTRUCTURE ONLY -- empty stand-in: the reference GPU sources include this header but use nothing from it. */
